// SPDX-License-Identifier: Apache-2.0
// ZeRO-style sharded optimizer and symmetric-memory flattening. See cs/parallel.h.
#include "cs/parallel.h"

#include <c10/cuda/CUDAStream.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <unordered_map>

#include "kernels/collectives.h"
#include "symm_internal.h"

namespace cs::parallel {
using communication::SymmetricContext;

std::shared_ptr<module::FlatParameters> flatten_symmetric(const Scheduler &scheduler, const module::Module &module,
                                                         const communication::Comm &comm, optional<at::ScalarType> lp_dtype,
                                                         const std::vector<std::string> &first, bool unequal_shards) {
  auto ctx = comm.impl()->symmetric;
  module::FlattenOptions opts;
  opts.lp_dtype(lp_dtype).transposed_copies(false).pad_total_to(comm.get_size() * 128).first(first);
  if (ctx) {
    // Symmetric memory only works while every rank allocates the same sizes in the same order: a buffer's offset is
    // its address on every peer. The arenas of a module whose shards differ in size between ranks (20 heads over 8
    // ranks) would shift everything allocated after them, so with `unequal_shards` each allocation takes the largest
    // size any rank asks for. Replicas (data parallel, sharded optimizer) have equal sizes and skip the round trip.
    static std::atomic<int64_t> calls{0};
    const std::string prefix = str_cat("cs/flatten_symmetric/", calls.fetch_add(1), "/");
    auto serial = std::make_shared<int>(0);
    auto store = unequal_shards ? comm.impl()->store : c10::intrusive_ptr<c10d::Store>{};
    opts.arena_allocator([ctx, store, prefix, serial, rank = comm.get_rank(), size = comm.get_size()](int64_t bytes) {
      const int64_t agreed = agree_on_max(store.get(), str_cat(prefix, (*serial)++, "/"), rank, size, bytes);
      const auto block = ctx->allocate(agreed);
      return ctx->tensor(block, {bytes}, at::kByte);
    });
  }
  return module::flatten_parameters(scheduler, module, opts);
}

int64_t agree_on_max(c10d::Store *store, const std::string &prefix, int rank, int size, int64_t value) {
  if (size <= 1 || store == nullptr) return value;
  const std::string mine = std::to_string(value);
  store->set(str_cat(prefix, rank), std::vector<uint8_t>(mine.begin(), mine.end()));
  int64_t agreed = value;
  for (int p = 0; p < size; ++p) {
    const auto raw = store->get(str_cat(prefix, p));  // blocks until that rank has published (store timeout applies)
    agreed = std::max<int64_t>(agreed, std::stoll(std::string(raw.begin(), raw.end())));
  }
  return agreed;
}

ZeroAdamWImpl::ZeroAdamWImpl(const Scheduler &scheduler, const module::Module &module,
                             const std::shared_ptr<module::FlatParameters> &flat, const communication::Comm &comm,
                             const Options &options)
    : flat_{flat}, comm_{comm} {
  bind(&module);
  flat->params.wait();
  CS_ASSERT_TRUE(flat->params.impl()->tensor.scalar_type() == at::kFloat, "ZeroAdamW needs fp32 master parameters");
  const int64_t world = comm.get_size(), rank = comm.get_rank();
  // Ownership of the arena is interleaved in blocks: block j belongs to rank j % world. This rank's shard holds its
  // blocks back to back (whole blocks; the last one may reach past the arena's end and is then partly unused).
  const int64_t blocks = (flat->total + kBlock - 1) / kBlock;
  const int64_t mine = blocks > rank ? (blocks - rank + world - 1) / world : 0;
  shard_count_ = std::max<int64_t>((blocks + world - 1) / world, 1) * kBlock;  // the same length on every rank
  Tensor shard;
  submit(scheduler, "cs::parallel::ZeroAdamW::shard_master", Task::Impl::kMain, Task::Impl::kCompute, {shard}, {flat->params},
         [shard, flat, rank, world, mine, n = shard_count_](const FnTask &) {
           const at::Tensor &P = flat->params.impl()->tensor;
           at::Tensor w = at::zeros({n}, P.options());
           for (int64_t k = 0; k < mine; ++k) {  // copy block rank + k * world
             const int64_t begin = (rank + k * world) * kBlock;
             const int64_t len = std::min<int64_t>(kBlock, flat->total - begin);
             if (len > 0) w.narrow(0, k * kBlock, len).copy_(P.narrow(0, begin, len));
           }
           shard.impl()->tensor = w;
         });
  master_ = shard;
  state_ = optimizer::AdamW::init(scheduler, shard, options);
  states_.insert("__shard__", state_);
  auto named = module.named_parameters();
  for (size_t i = 0; i < flat->slots.size(); ++i) {
    slot_params_.push_back(named[flat->slots[i].key]);
    slot_of_grad_.emplace(flat->grad_handles[i].impl().get(), i);
  }
}

OrderedDict<std::string, Tensor> ZeroAdamWImpl::named_state_tensors() const {
  OrderedDict<std::string, Tensor> out;
  out.insert(str_cat("shard", comm_.get_rank(), ".m"), state_->tensors.m);
  out.insert(str_cat("shard", comm_.get_rank(), ".v"), state_->tensors.v);
  out.insert(str_cat("shard", comm_.get_rank(), ".master"), master_);
  return out;
}

void ZeroAdamWImpl::step_partial(const Scheduler &scheduler, const std::vector<Tensor> &gradients, Task::Impl::Priority priority) {
  const module::Module *m = model();
  CS_ASSERT_TRUE(m != nullptr, "the optimised module is gone");
  if (!step_open_) {
    step_open_ = true;
    ++state_->options.t;
    slot_done_.assign(flat_->slots.size(), 0);
  }
  std::vector<size_t> picked;
  for (auto &g : gradients) {
    auto it = slot_of_grad_.find(g.impl().get());
    if (it == slot_of_grad_.end() || slot_done_[it->second]) continue;
    slot_done_[it->second] = 1;
    picked.push_back(it->second);
  }
  if (picked.empty()) return;
  std::sort(picked.begin(), picked.end());
  struct Range {
    int64_t begin, end;
  };
  std::vector<Range> ranges;  // runs of neighbouring slots are contiguous in the arenas (padding included)
  std::vector<Tensor> outs;
  std::vector<ReadOnlyTensor> ins;
  auto slot_end = [&](size_t i) { return i + 1 < flat_->slots.size() ? flat_->slots[i + 1].offset : flat_->total; };
  for (size_t k = 0; k < picked.size(); ++k) {
    const size_t i = picked[k];
    if (k > 0 && picked[k - 1] + 1 == i)
      ranges.back().end = slot_end(i);
    else
      ranges.push_back({flat_->slots[i].offset, slot_end(i)});
    outs.push_back(slot_params_[i]);
    ins.push_back(flat_->grad_handles[i]);
  }
  outs.push_back(master_);
  outs.push_back(state_->tensors.m);
  outs.push_back(state_->tensors.v);
  auto ctx = comm_.impl()->symmetric;
  const int64_t t = state_->options.t;
  submit(scheduler, "cs::parallel::ZeroAdamW::step(reduce-scatter + AdamW + all-gather)", priority, Task::Impl::kNccl, outs, ins,
         [flat = flat_, state = state_, master = master_, ctx, t, ranges, handles = ins, world = comm_.get_size(),
          touched = std::vector<Tensor>(outs.begin(), outs.end() - 3)](const FnTask &) {
           const auto &o = state->options;
           const double bc1 = 1.0 - std::pow(o.beta1, static_cast<double>(t));
           const double bc2 = 1.0 - std::pow(o.beta2, static_cast<double>(t));
           at::Tensor &G = flat->grads.impl()->tensor;
           at::Tensor &L = flat->lp.impl()->tensor;
           at::Tensor &W = master.impl()->tensor;
           for (auto &h : handles)  // a slot nobody wrote this step must not contribute stale values
             if (h.impl()->fresh && h.impl()->tensor.defined()) const_cast<at::Tensor &>(h.impl()->tensor).zero_();
           if (ctx && W.is_cuda() && world > 1) {
             int64_t g_off = 0, l_off = -1;
             CS_ASSERT_TRUE(ctx->locate(G.data_ptr(), static_cast<int64_t>(G.nbytes()), &g_off),
                            "ZeroAdamW needs the gradient arena in symmetric memory (use flatten_symmetric)");
             if (L.defined())
               CS_ASSERT_TRUE(ctx->locate(L.data_ptr(), static_cast<int64_t>(L.nbytes()), &l_off),
                              "ZeroAdamW needs the bf16 arena in symmetric memory (use flatten_symmetric)");
             const kernels::PeerTable table = communication::table_of(*ctx);
             for (auto &r : ranges) {
               kernels::ShardedAdamWArgs a{};
               a.grad_offset_bytes = g_off;
               a.lp_offset_bytes = l_off;
               a.master = W.data_ptr<float>();
               a.exp_avg = state->tensors.m.impl()->tensor.data_ptr<float>();
               a.exp_avg_sq = state->tensors.v.impl()->tensor.data_ptr<float>();
               a.range_begin = r.begin;
               a.range_end = r.end;
               a.block = kBlock;
               a.lr = static_cast<float>(o.lr);
               a.beta1 = static_cast<float>(o.beta1);
               a.beta2 = static_cast<float>(o.beta2);
               a.eps = static_cast<float>(o.eps);
               a.weight_decay = static_cast<float>(o.weight_decay);
               a.inv_bias_correction1 = static_cast<float>(1.0 / bc1);
               a.inv_bias_correction2 = static_cast<float>(1.0 / bc2);
               a.grad_scale = static_cast<float>(o.grad_scale / static_cast<double>(world));
               a.clip_coef = state->clip_coef.impl()->tensor.defined() ? state->clip_coef.impl()->tensor.data_ptr<float>() : nullptr;
               // one launch: "every rank's gradients of this range are complete" and "every rank's bf16 arena received
               // the updated range" are the barriers at the two ends of the kernel
               int blocks = 0;
               const auto h = communication::begin_collective(*ctx, kernels::kChanZero);
               const int code = kernels::symm_reduce_scatter_adamw_all_gather(c10::cuda::getCurrentCUDAStream().stream(), table, h, a, &blocks);
               CS_ASSERT_TRUE(code == 0, "fused reduce-scatter/AdamW/all-gather launch failed: ", cuda_error_string(code));
               communication::end_collective(*ctx, kernels::kChanZero, blocks);
             }
           } else {
             // Single rank (or CPU): the same update on the whole range (the shard is the arena, block by block).
             CS_ASSERT_TRUE(world == 1, "ZeroAdamW across ranks needs symmetric memory on CUDA devices");
             at::Tensor mm = state->tensors.m.impl()->tensor, vv = state->tensors.v.impl()->tensor;
             for (auto &r : ranges) {
               const int64_t n = r.end - r.begin;
               at::Tensor g = G.narrow(0, r.begin, n).to(at::kFloat) * o.grad_scale;
               at::Tensor w = W.narrow(0, r.begin, n), m1 = mm.narrow(0, r.begin, n), v1 = vv.narrow(0, r.begin, n);
               w.mul_(1 - o.lr * o.weight_decay);
               m1.mul_(o.beta1).add_(g, 1 - o.beta1);
               v1.mul_(o.beta2).addcmul_(g, g, 1 - o.beta2);
               w.sub_((m1 / bc1) / ((v1 / bc2).sqrt() + o.eps) * o.lr);
               if (L.defined()) L.narrow(0, r.begin, n).copy_(w);
               flat->params.impl()->tensor.narrow(0, r.begin, n).copy_(w);
             }
           }
           for (auto &p : touched) {
             auto &impl = *p.impl();
             ++impl.version;
             if (impl.lp.defined()) impl.lp_version = impl.version;
             if (impl.lp_t.defined()) {
               // the transpose is rebuilt from the fresh bf16 copy (the fp32 arena is not kept current between
               // gather_master calls)
               impl.lp_t.copy_(impl.lp.t());
               impl.lp_t_version = impl.version;
             }
           }
         });
}

void ZeroAdamWImpl::step(const Scheduler &scheduler) {
  // update whatever the buckets have not handed over yet (everything, when no bucket drives this optimizer)
  std::vector<Tensor> rest;
  if (!step_open_) {
    rest.assign(flat_->grad_handles.begin(), flat_->grad_handles.end());
  } else {
    for (size_t i = 0; i < flat_->slots.size(); ++i)
      if (!slot_done_[i]) rest.push_back(flat_->grad_handles[i]);
  }
  step_partial(scheduler, rest, Task::Impl::kComm);
  step_open_ = false;
}

void ZeroAdamWImpl::gather_master(const Scheduler &scheduler) {
  const int64_t world = comm_.get_size();
  if (world <= 1) return;
  std::vector<Tensor> recv(static_cast<size_t>(world));
  Tensor gathered;
  std::vector<Tensor> outs = recv;
  outs.push_back(gathered);
  submit(scheduler, "cs::parallel::ZeroAdamW::gather_buffers", Task::Impl::kMain, Task::Impl::kCompute, outs, {master_},
         [recv, gathered, master = master_, world](const FnTask &) {
           const at::Tensor &w = master.impl()->tensor;
           gathered.impl()->tensor = at::empty({world, w.numel()}, w.options());
           for (size_t r = 0; r < recv.size(); ++r) recv[r].impl()->tensor = gathered.impl()->tensor.select(0, static_cast<int64_t>(r));
         });
  communication::AllGather::run(scheduler, comm_, {recv}, {master_});
  std::vector<ReadOnlyTensor> ins(recv.begin(), recv.end());
  ins.push_back(gathered);
  submit(scheduler, "cs::parallel::ZeroAdamW::unshard_master", Task::Impl::kComm, Task::Impl::kCompute, {flat_->params}, ins,
         [flat = flat_, gathered, world](const FnTask &) {
           // [world, blocks_per_rank, block] -> arena order [blocks_per_rank, world, block]
           const at::Tensor &g = gathered.impl()->tensor;
           const int64_t per = g.size(1) / kBlock;
           at::Tensor ordered = g.view({world, per, kBlock}).permute({1, 0, 2}).reshape({-1});
           at::Tensor &P = flat->params.impl()->tensor;
           P.copy_(ordered.narrow(0, 0, P.numel()));
         });
}

// ======================================================================================
// Tensor parallel GPT-2
// ======================================================================================
Tensor all_gather_rows(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &shard) {
  const int64_t world = comm.get_size();
  if (world <= 1) {
    Tensor same;
    submit(scheduler, "cs::parallel::all_gather_rows", Task::Impl::kMain, Task::Impl::kCompute, {same}, {shard},
           [same, shard](const FnTask &) { same.impl()->tensor = shard.impl()->tensor; });
    return same;
  }
  Tensor full;
  std::vector<Tensor> parts(static_cast<size_t>(world));
  std::vector<Tensor> outs{full};
  outs.insert(outs.end(), parts.begin(), parts.end());
  submit(scheduler, "cs::parallel::all_gather_rows::allocate", Task::Impl::kMain, Task::Impl::kCompute, outs, {shard},
         [full, parts, shard, world](const FnTask &) {
           const at::Tensor &s = shard.impl()->tensor;
           auto sizes = s.sizes().vec();
           const int64_t rows = sizes[0];
           sizes[0] = rows * world;
           full.impl()->tensor = at::empty(sizes, s.options());
           for (int64_t r = 0; r < world; ++r) parts[r].impl()->tensor = full.impl()->tensor.narrow(0, r * rows, rows);
         });
  communication::AllGather::run(scheduler, comm, {parts}, {shard});
  // The gather wrote through the row views; tie the result handle to the comm-stream work.
  Tensor joined;
  std::vector<ReadOnlyTensor> deps(parts.begin(), parts.end());
  deps.push_back(full);
  submit(scheduler, "cs::parallel::all_gather_rows::join", Task::Impl::kComm, Task::Impl::kCompute, {joined}, deps,
         [joined, full](const FnTask &) { joined.impl()->tensor = full.impl()->tensor; });
  return joined;
}

Tensor reduce_scatter_rows(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &full,
                           const ReadOnlyTensor *residual) {
  const int64_t world = comm.get_size();
  const int64_t rank = comm.get_rank();
  Tensor out;
  if (world <= 1) {
    std::vector<ReadOnlyTensor> ins{full};
    std::optional<ReadOnlyTensor> res;
    if (residual) {
      res = *residual;
      ins.push_back(*residual);
    }
    submit(scheduler, "cs::parallel::reduce_scatter_rows", Task::Impl::kMain, Task::Impl::kCompute, {out}, ins,
           [out, full, res](const FnTask &) {
             out.impl()->tensor = res ? full.impl()->tensor + res->impl()->tensor : full.impl()->tensor;
           });
    return out;
  }
  std::vector<Tensor> parts(static_cast<size_t>(world));
  Tensor recv;
  std::vector<Tensor> outs{recv};
  outs.insert(outs.end(), parts.begin(), parts.end());
  submit(scheduler, "cs::parallel::reduce_scatter_rows::views", Task::Impl::kMain, Task::Impl::kCompute, outs, {full},
         [recv, parts, full, world](const FnTask &) {
           const at::Tensor &f = full.impl()->tensor;
           CS_ASSERT_TRUE(f.size(0) % world == 0, "row count ", f.size(0), " does not split over ", world, " ranks");
           const int64_t rows = f.size(0) / world;
           for (int64_t r = 0; r < world; ++r) parts[r].impl()->tensor = f.narrow(0, r * rows, rows);
           auto sizes = f.sizes().vec();
           sizes[0] = rows;
           recv.impl()->tensor = at::empty(sizes, f.options());
         });
  std::vector<ReadOnlyTensor> send(parts.begin(), parts.end());
  communication::ReduceScatter::run(scheduler, comm, {recv}, {send}, communication::kSUM);
  (void)rank;
  if (!residual) return recv;
  return compute::Utils::add(scheduler, recv, *residual);
}

// -------------------------------------------------- tensor-parallel collectives on symmetric memory ----
// Every gather / reduce-scatter below is ONE light kernel on the main stream (the barriers are inside it,
// kernels/collectives.h). Gathered activations live in persistent symmetric buffers, one pair per block,
// so the backward pass reads them again for the weight gradients instead of gathering a second time.
// Partial products of the row-parallel GEMMs are written (by the GEMM's own TMA-store epilogue) into one
// symmetric bf16 buffer; the owner of each row block then loads the sum over all ranks, reduced inside the
// switch when the arena has a multicast mapping, adds the residual and keeps its rows.
namespace {
std::atomic<int64_t> g_fused_tp_launches{0};

at::Tensor symmetric_tensor(communication::SymmetricContext &ctx, at::IntArrayRef sizes, at::ScalarType dtype) {
  int64_t numel = 1;
  for (auto v : sizes) numel *= v;
  return ctx.tensor(ctx.allocate(numel * static_cast<int64_t>(c10::elementSize(dtype))), sizes, dtype);
}

// (Re)creates the symmetric buffer behind `handle` when the shape changed. Called inside a task that lists
// `handle` as an output, on every rank in the same order, so the offsets agree.
at::Tensor &ensure_symmetric(communication::SymmetricContext &ctx, const Tensor &handle, at::IntArrayRef sizes, at::ScalarType dtype) {
  at::Tensor &t = handle.impl()->tensor;
  if (!t.defined() || t.sizes() != sizes || t.scalar_type() != dtype) {
    if (t.defined()) {
      int64_t off = 0;
      if (ctx.locate(t.data_ptr(), static_cast<int64_t>(t.nbytes()), &off))
        ctx.release(communication::SymmetricBlock{off, (static_cast<int64_t>(t.nbytes()) + 255) / 256 * 256});
    }
    t = symmetric_tensor(ctx, sizes, dtype);
  }
  return t;
}

bool fused_tp_ok(const communication::Comm &comm, const at::Tensor &x, int64_t total_rows) {
  auto ctx = comm.impl()->symmetric;
  const int64_t tp = comm.get_size();
  return ctx && tp > 1 && tp <= kernels::kMaxPeers && x.is_cuda() && x.scalar_type() == at::kBFloat16 &&
         compute::get_backend() == compute::Backend::kFused && total_rows % tp == 0 && x.size(-1) % 8 == 0;
}

// [m, k] row shard -> `full` [tp * m, k] on every rank (persistent symmetric buffer behind the handle).
void gather_rows_symmetric(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &shard, const Tensor &full) {
  submit(scheduler, "cs::parallel::gather_rows(symmetric push)", Task::Impl::kMain, Task::Impl::kCompute, {full}, {shard},
         [shard, full, comm](const FnTask &) {
           auto &ctx = *comm.impl()->symmetric;
           const at::Tensor xs = shard.impl()->tensor.reshape({-1, shard.impl()->tensor.size(-1)}).contiguous();
           const int64_t m = xs.size(0), k = xs.size(1), tp = ctx.size;
           at::Tensor &dst = ensure_symmetric(ctx, full, {m * tp, k}, xs.scalar_type());
           int64_t off = 0;
           CS_ASSERT_TRUE(ctx.locate(dst.data_ptr(), static_cast<int64_t>(dst.nbytes()), &off), "gather buffer left the arena");
           int blocks = 0;
           const auto h = communication::begin_collective(ctx, kernels::kChanGatherRows);
           const int code = kernels::symm_all_gather_push(c10::cuda::getCurrentCUDAStream().stream(), communication::table_of(ctx), h,
                                                          xs.data_ptr(), off, static_cast<int64_t>(xs.nbytes()), &blocks);
           CS_ASSERT_TRUE(code == 0, "row gather launch failed: ", cuda_error_string(code));
           communication::end_collective(ctx, kernels::kChanGatherRows, blocks);
           g_fused_tp_launches.fetch_add(1);
         });
}

// y[M, n] = x[M, k] * W^T (weight_is_rhs == false, W [n, k]) or x * W (true, W [k, n]) written into the symmetric
// `partial` buffer, then out[m, n] = sum over ranks of this rank's rows (+ residual): two launches, GEMM and
// reduce-scatter, both on the main stream.
Tensor row_parallel_symmetric(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &weight,
                              const ReadOnlyTensor &x, const ReadOnlyTensor *residual_shard, bool weight_is_rhs, const Tensor &partial) {
  Tensor out;
  std::vector<ReadOnlyTensor> ins{x, weight};
  std::optional<ReadOnlyTensor> res;
  if (residual_shard) {
    res = *residual_shard;
    ins.push_back(*residual_shard);
  }
  submit(scheduler, "cs::parallel::row_parallel(GEMM + switch reduce-scatter)", Task::Impl::kMain, Task::Impl::kCompute, {out, partial}, ins,
         [out, partial, x, weight, res, comm, weight_is_rhs](const FnTask &) {
           auto &ctx = *comm.impl()->symmetric;
           const int64_t tp = ctx.size;
           const at::Tensor xa = x.impl()->tensor.reshape({-1, x.impl()->tensor.size(-1)}).contiguous();
           const at::Tensor wc = compute::working_copy(weight, at::kBFloat16);
           const int64_t m = xa.size(0), k = xa.size(1);
           const int64_t n = weight_is_rhs ? wc.size(1) : wc.size(0);
           CS_ASSERT_TRUE(m % tp == 0, "row count ", m, " does not split over ", tp, " ranks");
           const int64_t rows = m / tp;
           at::Tensor &y = ensure_symmetric(ctx, partial, {m, n}, at::kBFloat16);
           auto stream = c10::cuda::getCurrentCUDAStream().stream();
           kernels::GemmArgs g{};
           g.a = xa.data_ptr();
           g.b = wc.data_ptr();
           g.d = y.data_ptr();
           g.m = m;
           g.n = n;
           g.k = k;
           g.lda = k;
           g.ldb = weight_is_rhs ? n : k;
           g.ldd = n;
           g.layout = weight_is_rhs ? kernels::kTM : kernels::kTN;
           g.epilogue = kernels::kEpiStoreBf16;
           const int code = kernels::gemm_bf16(stream, g);
           CS_ASSERT_TRUE(code == 0, "row-parallel GEMM launch failed (", code, ") for m=", m, " n=", n, " k=", k);
           int64_t off = 0;
           CS_ASSERT_TRUE(ctx.locate(y.data_ptr(), static_cast<int64_t>(y.nbytes()), &off), "partial buffer left the arena");
           at::Tensor o = at::empty({rows, n}, xa.options());
           at::Tensor r;
           if (res) r = res->impl()->tensor.reshape({rows, n}).contiguous();
           int blocks = 0;
           const auto h = communication::begin_collective(ctx, kernels::kChanScatterRows);
           const int rc = kernels::symm_reduce_scatter(stream, communication::table_of(ctx), h, off + ctx.rank * rows * n * 2, o.data_ptr(),
                                                       rows * n, 1, 1.0f, &blocks, res ? r.data_ptr() : nullptr);
           CS_ASSERT_TRUE(rc == 0, "row reduce-scatter launch failed: ", cuda_error_string(rc));
           communication::end_collective(ctx, kernels::kChanScatterRows, blocks);
           g_fused_tp_launches.fetch_add(1);
           out.impl()->tensor = o;
         });
  return out;
}

}  // namespace

// ---- the fused kernels on plain tensors, for one rank, on the current stream ---------------------------------
GatherSignal gather_rows_chunked(communication::SymmetricContext &ctx, const at::Tensor &shard, const at::Tensor &full, int chunks) {
  CS_ASSERT_TRUE(shard.is_contiguous() && shard.dim() == 2 && full.dim() == 2 && full.size(0) == shard.size(0) * ctx.size &&
                     full.size(1) == shard.size(1) && full.scalar_type() == shard.scalar_type(),
                 "gather_rows_chunked: full must be [size * rows, k] of the shard's dtype");
  int64_t off = 0;
  CS_ASSERT_TRUE(ctx.locate(full.data_ptr(), static_cast<int64_t>(full.nbytes()), &off), "the gather buffer must live in the symmetric arena");
  int blocks = 0;
  const auto h = communication::begin_collective(ctx, kernels::kChanGemmGather);
  const int code = kernels::symm_all_gather_chunked(c10::cuda::getCurrentCUDAStream().stream(), communication::table_of(ctx), h, shard.data_ptr(),
                                                    off, static_cast<int64_t>(shard.nbytes()), chunks, &blocks);
  CS_ASSERT_TRUE(code == 0, "chunked row gather launch failed: ", cuda_error_string(code));
  communication::end_collective(ctx, kernels::kChanGemmGather, blocks);
  GatherSignal signal;
  signal.epoch = h.epoch;
  signal.flags = ctx.flags[ctx.rank] + kernels::kChannelBase + kernels::kChanGemmGather * kernels::kChannelWords + kernels::kChunkFlags;
  signal.chunks = chunks;
  return signal;
}

std::pair<at::Tensor, at::Tensor> gemm_on_gathered_chunks(communication::SymmetricContext &ctx, const at::Tensor &full, const at::Tensor &weight,
                                                          bool weight_is_rhs, int epilogue, const at::Tensor &aux, const GatherSignal &signal) {
  const int64_t m = full.size(0), k = full.size(1);
  const int64_t n = weight_is_rhs ? weight.size(1) : weight.size(0);
  at::Tensor y = at::empty({m, n}, full.options());
  at::Tensor y2, a2;
  kernels::GemmArgs g{};
  g.a = full.data_ptr();
  g.b = weight.data_ptr();
  g.d = y.data_ptr();
  g.m = m;
  g.n = n;
  g.k = k;
  g.lda = k;
  g.ldb = weight_is_rhs ? n : k;
  g.ldd = n;
  g.layout = weight_is_rhs ? kernels::kTM : kernels::kTN;
  g.epilogue = epilogue;
  if (epilogue == kernels::kEpiGeluDual) {
    y2 = at::empty_like(y);
    g.d2 = y2.data_ptr();
  }
  if (aux.defined()) {
    a2 = aux.reshape({m, n}).contiguous();
    g.aux = a2.data_ptr();
  }
  g.peer_count = ctx.size;
  g.peer_rank = ctx.rank;
  g.ready_flags = signal.flags;
  g.ready_epoch = signal.epoch;
  g.ready_chunks = signal.chunks;
  const int code = kernels::gemm_bf16(c10::cuda::getCurrentCUDAStream().stream(), g);
  CS_ASSERT_TRUE(code == 0, "GEMM on gathered chunks failed to launch (", code, ") for m=", m, " n=", n, " k=", k);
  return {y, y2};
}

void gemm_scatter_to_slots(communication::SymmetricContext &ctx, const at::Tensor &x, const at::Tensor &weight, bool weight_is_rhs,
                           const at::Tensor &slots) {
  const int64_t tp = ctx.size;
  const int64_t m = x.size(0), k = x.size(1);
  const int64_t n = weight_is_rhs ? weight.size(1) : weight.size(0);
  const int64_t rows = m / tp;
  CS_ASSERT_TRUE(x.is_contiguous() && m % tp == 0 && slots.dim() == 3 && slots.size(0) == tp && slots.size(1) == rows && slots.size(2) == n &&
                     slots.scalar_type() == at::kBFloat16,
                 "gemm_scatter_to_slots: slots must be bf16 [size, rows / size, n]");
  int64_t off = 0;
  CS_ASSERT_TRUE(ctx.locate(slots.data_ptr(), static_cast<int64_t>(slots.nbytes()), &off), "the slot buffer must live in the symmetric arena");
  kernels::GemmArgs g{};
  g.a = x.data_ptr();
  g.b = weight.data_ptr();
  g.m = m;
  g.n = n;
  g.k = k;
  g.lda = k;
  g.ldb = weight_is_rhs ? n : k;
  g.ldd = n;
  g.layout = weight_is_rhs ? kernels::kTM : kernels::kTN;
  g.epilogue = kernels::kEpiStoreBf16;
  g.peer_count = static_cast<int>(tp);
  g.peer_rank = ctx.rank;
  for (int p = 0; p < tp; ++p) g.d_peers[p] = ctx.bases[p] + off + static_cast<int64_t>(ctx.rank) * rows * n * 2;
  const int code = kernels::gemm_bf16(c10::cuda::getCurrentCUDAStream().stream(), g);
  CS_ASSERT_TRUE(code == 0, "GEMM with scatter epilogue failed to launch (", code, ") for m=", m, " n=", n, " k=", k);
}

at::Tensor sum_slots(communication::SymmetricContext &ctx, const at::Tensor &slots, const at::Tensor &residual) {
  const int64_t rows = slots.size(1), n = slots.size(2);
  at::Tensor o = at::empty({rows, n}, slots.options());
  at::Tensor r;
  if (residual.defined()) r = residual.reshape({rows, n}).contiguous();
  const auto h = communication::begin_collective(ctx, kernels::kChanGemmScatter);
  const int rc = kernels::symm_slot_sum(c10::cuda::getCurrentCUDAStream().stream(), communication::table_of(ctx), h, slots.data_ptr(), rows * n * 2,
                                        o.data_ptr(), residual.defined() ? r.data_ptr() : nullptr, rows * n);
  CS_ASSERT_TRUE(rc == 0, "slot sum launch failed: ", cuda_error_string(rc));
  return o;
}

namespace {
// ---- fused forms (row shards that are multiples of 256 rows) ------------------------------------------------
// all-gather -> GEMM: the gather runs on the communication stream in row chunks and announces every chunk with a
// flag; the GEMM on the main stream starts at once and its TMA producer waits for the flag of the chunk a tile
// needs, so the multiplication proceeds while later chunks are still crossing NVLink.
// GEMM -> reduce-scatter: the GEMM epilogue TMA-stores each bf16 output tile straight into the slot that the
// owner of those rows keeps for this rank; one kernel then opens with the cross-rank barrier and sums the local
// slots (+ residual). No barrier launches, no zero-filling, every byte crosses NVLink once as bf16.
int gather_chunks_for(int64_t rows_per_rank) {
  for (int c : {4, 2, 1})
    if (rows_per_rank % (256 * c) == 0) return c;
  return 0;
}

// y[M, n] = gather(x_shard)[M, k] * W^T (W [n, k]) or * W (weight_is_rhs, W [k, n]); `full` keeps the gathered rows.
// epilogue: kEpiStoreBf16, kEpiGeluDual (companion = GELU(y)) or kEpiDGelu (aux = pre-activation).
Tensor gather_gemm(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &x_shard, const Tensor &full,
                   const ReadOnlyTensor &weight, bool weight_is_rhs, int epilogue, const ReadOnlyTensor *aux) {
  const int chunks = gather_chunks_for(x_shard.impl()->tensor.numel() / x_shard.impl()->tensor.size(-1));
  auto signal = std::make_shared<GatherSignal>();
  submit(scheduler, "cs::parallel::gather_rows(chunked push beside the GEMM)", Task::Impl::kComm, Task::Impl::kNccl, {full}, {x_shard},
         [x_shard, full, comm, chunks, signal](const FnTask &task) {
           auto &ctx = *comm.impl()->symmetric;
           const at::Tensor xs = x_shard.impl()->tensor.reshape({-1, x_shard.impl()->tensor.size(-1)}).contiguous();
           task.intermediate().push_back(xs);
           at::Tensor &dst = ensure_symmetric(ctx, full, {xs.size(0) * ctx.size, xs.size(1)}, xs.scalar_type());
           *signal = gather_rows_chunked(ctx, xs, dst, chunks);
         });
  Tensor out;
  std::vector<ReadOnlyTensor> ins{x_shard, weight};  // not `full`: the flags order the reads, chunk by chunk
  std::optional<ReadOnlyTensor> aux_h;
  if (aux) {
    aux_h = *aux;
    ins.push_back(*aux);
  }
  submit(scheduler, "cs::parallel::column_parallel(GEMM on arriving chunks)", Task::Impl::kMain, Task::Impl::kCompute, {out}, ins,
         [out, full, weight, weight_is_rhs, epilogue, aux_h, comm, signal](const FnTask &task) {
           auto &ctx = *comm.impl()->symmetric;
           const at::Tensor wc = compute::working_copy(weight, at::kBFloat16);
           at::Tensor a2;
           if (aux_h) a2 = aux_h->impl()->tensor;
           auto [y, y2] = gemm_on_gathered_chunks(ctx, full.impl()->tensor, wc, weight_is_rhs, epilogue, a2, *signal);
           g_fused_tp_launches.fetch_add(1);
           out.impl()->tensor = y;
           out.impl()->companion = y2;
         });
  return out;
}

// out[m, n] = sum over ranks of (x * W^T or x * W)[rows of this rank] (+ residual): GEMM with the scatter in its epilogue,
// then the slot sum. `slots` are two symmetric buffers [tp, m, n] bf16 used in turn.
Tensor gemm_scatter(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &weight, const ReadOnlyTensor &x,
                    const ReadOnlyTensor *residual_shard, bool weight_is_rhs, TPWorkspace &ws) {
  Tensor out;
  const Tensor slots = ws.slots[ws.next_slot ^= 1];
  std::vector<ReadOnlyTensor> ins{x, weight};
  std::optional<ReadOnlyTensor> res;
  if (residual_shard) {
    res = *residual_shard;
    ins.push_back(*residual_shard);
  }
  submit(scheduler, "cs::parallel::row_parallel(GEMM with bf16 scatter epilogue + slot sum)", Task::Impl::kMain, Task::Impl::kCompute,
         {out, slots}, ins, [out, slots, x, weight, res, comm, weight_is_rhs](const FnTask &) {
           auto &ctx = *comm.impl()->symmetric;
           const int64_t tp = ctx.size;
           const at::Tensor xa = x.impl()->tensor.reshape({-1, x.impl()->tensor.size(-1)}).contiguous();
           const at::Tensor wc = compute::working_copy(weight, at::kBFloat16);
           const int64_t m = xa.size(0);
           const int64_t n = weight_is_rhs ? wc.size(1) : wc.size(0);
           const int64_t rows = m / tp;
           at::Tensor &buf = ensure_symmetric(ctx, slots, {tp, rows, n}, at::kBFloat16);  // slot s: rank s's partial of my rows
           gemm_scatter_to_slots(ctx, xa, wc, weight_is_rhs, buf);
           at::Tensor r;
           if (res) r = res->impl()->tensor;
           at::Tensor o = sum_slots(ctx, buf, r);
           g_fused_tp_launches.fetch_add(1);
           out.impl()->tensor = o;
         });
  return out;
}
}  // namespace

int64_t fused_tp_launches() { return g_fused_tp_launches.load(); }

namespace {
compute::Linear::Options tp_linear(const Scheduler &scheduler, const models::GPT2Config &c, int64_t in, int64_t out) {
  return compute::Linear::Options{in, out}.bias(false).device(c.device().value_or(scheduler.device())).dtype(c.dtype());
}
}  // namespace

TPBlockImpl::TPBlockImpl(const Scheduler &scheduler, const models::GPT2Config &config, const communication::Comm &comm_)
    : comm{comm_} {
  const int64_t tp = comm.get_size();
  const int64_t d = config.n_embd();
  const int64_t rank = comm.get_rank();
  CS_ASSERT_TRUE(config.n_head() >= tp, "n_head (", config.n_head(), ") is smaller than the tensor-parallel size ", tp);
  CS_ASSERT_TRUE(d % config.n_head() == 0 && (4 * d) % tp == 0, "n_embd must be a multiple of n_head, and 4*n_embd of the tensor-parallel size");
  const int64_t head_dim = d / config.n_head(), extra = config.n_head() % tp;
  local_heads = config.n_head() / tp + (rank < extra ? 1 : 0);
  head_begin = rank * (config.n_head() / tp) + std::min<int64_t>(rank, extra);
  const int64_t d_attn = local_heads * head_dim;  // this rank's slice of the attention width
  auto ln_opts = compute::LayerNorm::Options{d}.device(config.device().value_or(scheduler.device())).dtype(config.dtype());
  ln1 = register_module("ln1", module::LayerNorm{scheduler, ln_opts});
  c_attn = register_module("c_attn", module::Linear{scheduler, tp_linear(scheduler, config, d, 3 * d_attn)});
  c_proj = register_module("c_proj", module::Linear{scheduler, tp_linear(scheduler, config, d_attn, d)});
  ln2 = register_module("ln2", module::LayerNorm{scheduler, ln_opts});
  fc1 = register_module("fc1", module::Linear{scheduler, tp_linear(scheduler, config, d, 4 * d / tp).gelu_epilogue(true)});
  fc2 = register_module("fc2", module::GeluLinear{scheduler, tp_linear(scheduler, config, 4 * d / tp, d)});
  attn_state = compute::ScaledDotProductAttention::init(scheduler, compute::ScaledDotProductAttention::Options{}.is_causal(true));
  for (auto *w : {&c_attn->state()->forward.weight, &c_proj->state()->forward.weight, &fc1->state()->forward.weight})
    compute::Utils::normal_(scheduler, *w, 0, config.init_std());
  compute::Utils::normal_(scheduler, fc2->state()->forward.weight, 0, config.init_std());
}

Tensor TPBlockImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &x_shard, int64_t batch, int64_t seq) {
  namespace Utils = compute::Utils;
  const int64_t d_local = c_proj->state()->forward.weight.size(1);
  const bool fuse = workspace && x_shard.defined() && fused_tp_ok(comm, x_shard.impl()->tensor, batch * seq) &&
                    scheduler.impl()->autocast_enabled;
  fused_forward_ = fuse;
  // row shards of whole 256-row tiles take the fused kernels (gather beside the GEMM, scatter in the GEMM epilogue)
  const bool tiles = fuse && (batch * seq / comm.get_size()) % 256 == 0;
  tiled_forward_ = tiles;
  auto mark_bf16 = [](const Tensor &w) {
    w.impl()->autocast_enabled = true;
    w.impl()->autocast_dtype = at::kBFloat16;
  };
  Tensor a = ln1->forward(scheduler, x_shard);                 // [M/tp, d]
  Tensor qkv;                                                   // [M, 3 d/tp]
  if (tiles) {
    mark_bf16(c_attn->state()->forward.weight);
    qkv = gather_gemm(scheduler, comm, a, a_full, c_attn->state()->forward.weight, false, kernels::kEpiStoreBf16, nullptr);
    c_attn->state()->backward.input = a_full;                  // kept: the weight gradient of c_attn reads it again
  } else if (fuse) {
    gather_rows_symmetric(scheduler, comm, a, a_full);
    qkv = c_attn->forward(scheduler, a_full);
  } else {
    qkv = c_attn->forward(scheduler, all_gather_rows(scheduler, comm, a));
  }
  Tensor qkv3 = Utils::view(scheduler, qkv, {batch, seq, 3 * d_local});
  Tensor ctx = compute::ScaledDotProductAttention::forward_packed(scheduler, attn_state, qkv3, local_heads);
  Tensor ctx2 = Utils::view(scheduler, ctx, {batch * seq, d_local});
  Tensor x1;                                                     // [M/tp, d] + residual
  if (fuse) {
    c_proj->state()->backward.input = ctx2;
    c_proj->state()->forward.weight.impl()->autocast_enabled = true;
    c_proj->state()->forward.weight.impl()->autocast_dtype = at::kBFloat16;
    x1 = tiles ? gemm_scatter(scheduler, comm, c_proj->state()->forward.weight, ctx2, &x_shard, false, *workspace)
               : row_parallel_symmetric(scheduler, comm, c_proj->state()->forward.weight, ctx2, &x_shard, false, workspace->partial);
  } else {
    x1 = reduce_scatter_rows(scheduler, comm, c_proj->forward(scheduler, ctx2), &x_shard);
  }
  Tensor b = ln2->forward(scheduler, x1);
  Tensor pre;                                                    // [M, 4d/tp], carries GELU
  if (tiles) {
    mark_bf16(fc1->state()->forward.weight);
    pre = gather_gemm(scheduler, comm, b, b_full, fc1->state()->forward.weight, false, kernels::kEpiGeluDual, nullptr);
    fc1->state()->backward.input = b_full;
  } else if (fuse) {
    gather_rows_symmetric(scheduler, comm, b, b_full);
    pre = fc1->forward(scheduler, b_full);
  } else {
    pre = fc1->forward(scheduler, all_gather_rows(scheduler, comm, b));
  }
  if (!fuse) return reduce_scatter_rows(scheduler, comm, fc2->forward(scheduler, pre), &x1);
  // fc2 consumes GELU(pre), the companion emitted by the fc1 epilogue
  Tensor act;
  submit(scheduler, "cs::parallel::TPBlock::activation_view", Task::Impl::kMain, Task::Impl::kCompute, {act}, {pre},
         [act, pre](const FnTask &) { act.impl()->tensor = pre.impl()->companion; });
  auto fs = fc2->state();
  fs->backward.input = pre;
  fs->backward.activated = act;
  fs->backward.input_count = 2;
  fs->forward.weight.impl()->autocast_enabled = true;
  fs->forward.weight.impl()->autocast_dtype = at::kBFloat16;
  return tiles ? gemm_scatter(scheduler, comm, fs->forward.weight, act, &x1, false, *workspace)
               : row_parallel_symmetric(scheduler, comm, fs->forward.weight, act, &x1, false, workspace->partial);
}

Tensor TPBlockImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_shard, const models::GradientSync &sync) {
  namespace Utils = compute::Utils;
  const bool fuse = fused_forward_, tiles = tiled_forward_;
  // MLP: reduce-scatter backward = all-gather of the incoming row shard
  Tensor dz, d_pre;                                              // [M, d], [M, 4d/tp]
  if (tiles) {
    dz = workspace->grad_full[workspace->next_grad ^= 1];
    auto fs = fc2->state();
    const ReadOnlyTensor pre = fs->backward.input;
    d_pre = gather_gemm(scheduler, comm, grad_shard, dz, fs->forward.weight, true, kernels::kEpiDGelu, &pre);  // includes GELU'
    fs->backward.input_count = 1;                                // the input-gradient half ran here
  } else {
    if (fuse) {
      dz = workspace->grad_full[workspace->next_grad ^= 1];
      gather_rows_symmetric(scheduler, comm, grad_shard, dz);
    } else {
      dz = all_gather_rows(scheduler, comm, grad_shard);
    }
    d_pre = fc2->backward_input(scheduler, dz);
  }
  fc2->backward_parameter(scheduler, dz);
  Tensor d_b;                                                    // all-gather backward = reduce-scatter
  if (tiles) {
    d_b = gemm_scatter(scheduler, comm, fc1->state()->forward.weight, d_pre, nullptr, true, *workspace);
  } else if (fuse) {
    d_b = row_parallel_symmetric(scheduler, comm, fc1->state()->forward.weight, d_pre, nullptr, true, workspace->partial);
  } else {
    d_b = reduce_scatter_rows(scheduler, comm, fc1->backward_input(scheduler, d_pre));
  }
  fc1->backward_parameter(scheduler, d_pre);                     // input: the gathered rows kept by forward
  Tensor d_x1 = ln2->backward(scheduler, d_b, grad_shard);       // + residual branch
  sync.push(scheduler, ln2->state()->forward.grad_weight);
  sync.push(scheduler, ln2->state()->forward.grad_bias);
  // attention
  Tensor dy, d_ctx;                                              // [M, d], [M, d/tp]
  if (tiles) {
    dy = workspace->grad_full[workspace->next_grad ^= 1];
    d_ctx = gather_gemm(scheduler, comm, d_x1, dy, c_proj->state()->forward.weight, true, kernels::kEpiStoreBf16, nullptr);
  } else {
    if (fuse) {
      dy = workspace->grad_full[workspace->next_grad ^= 1];
      gather_rows_symmetric(scheduler, comm, d_x1, dy);
    } else {
      dy = all_gather_rows(scheduler, comm, d_x1);
    }
    d_ctx = c_proj->backward_input(scheduler, dy);
  }
  c_proj->backward_parameter(scheduler, dy);
  Tensor d_qkv = compute::ScaledDotProductAttention::backward_packed(scheduler, attn_state, d_ctx);
  const int64_t three_d_local = c_attn->state()->forward.weight.size(0);
  Tensor d_qkv2 = Utils::view(scheduler, d_qkv, {-1, three_d_local});
  Tensor d_a;
  if (tiles) {
    d_a = gemm_scatter(scheduler, comm, c_attn->state()->forward.weight, d_qkv2, nullptr, true, *workspace);
  } else if (fuse) {
    d_a = row_parallel_symmetric(scheduler, comm, c_attn->state()->forward.weight, d_qkv2, nullptr, true, workspace->partial);
  } else {
    d_a = reduce_scatter_rows(scheduler, comm, c_attn->backward_input(scheduler, d_qkv2));
  }
  c_attn->backward_parameter(scheduler, d_qkv2);
  Tensor d_x = ln1->backward(scheduler, d_a, d_x1);
  sync.push(scheduler, ln1->state()->forward.grad_weight);
  sync.push(scheduler, ln1->state()->forward.grad_bias);
  return d_x;
}

TPGPT2Impl::TPGPT2Impl(const Scheduler &scheduler, const models::GPT2Config &config, const communication::Comm &comm)
    : config_{config}, comm_{comm} {
  const auto dev = config.device().value_or(scheduler.device());
  const int64_t d = config.n_embd();
  const int64_t tp = comm.get_size();
  wte = register_module("wte", module::Embedding{scheduler, compute::Embedding::Options{config.padded_vocab_size(), d}.device(dev).dtype(config.dtype())});
  wpe = register_module("wpe", module::Embedding{scheduler, compute::Embedding::Options{config.block_size(), d}.device(dev).dtype(config.dtype())});
  compute::Utils::normal_(scheduler, wte->state()->forward.weight, 0, config.init_std());
  compute::Utils::normal_(scheduler, wpe->state()->forward.weight, 0, config.init_std());
  auto workspace = std::make_shared<TPWorkspace>();
  for (int64_t l = 0; l < config.n_layer(); ++l) {
    h.push_back(register_module(std::to_string(l), TPBlock{scheduler, config, comm}));
    h.back()->workspace = workspace;
  }
  workspace_ = workspace;
  lnf = register_module("lnf", module::LayerNorm{scheduler, compute::LayerNorm::Options{d}.device(dev).dtype(config.dtype())});
  // The classifier is split over the vocabulary when it divides evenly (rows [rank * V/tp, (rank+1) * V/tp) of
  // lm_head live here); otherwise every rank keeps the whole matrix and scores its own token rows.
  vocab_parallel_ = tp > 1 && config.padded_vocab_size() % (tp * 8) == 0;
  const int64_t classes = vocab_parallel_ ? config.padded_vocab_size() / tp : config.padded_vocab_size();
  lm_head = register_module("lm_head", module::Linear{scheduler, compute::Linear::Options{d, classes}.bias(false).device(dev).dtype(config.dtype())});
  compute::Utils::normal_(scheduler, lm_head->state()->forward.weight, 0, config.init_std());
  lce_state_ = compute::LinearCrossEntropy::init(scheduler, lm_head->state(), config.vocab_size(), -100);
}

std::vector<std::string> TPGPT2Impl::replicated_parameters() const {
  std::vector<std::string> out{"wte.weight", "wpe.weight", "lnf.weight", "lnf.bias"};
  if (!vocab_parallel_) out.push_back("lm_head.weight");
  for (size_t l = 0; l < h.size(); ++l)
    for (const char *k : {".ln1.weight", ".ln1.bias", ".ln2.weight", ".ln2.bias"}) out.push_back(std::to_string(l) + k);
  return out;
}

Tensor TPGPT2Impl::forward_loss(const Scheduler &scheduler, const ReadOnlyTensor &input_ids, const ReadOnlyTensor &labels) {
  namespace Utils = compute::Utils;
  CS_ASSERT_TRUE(input_ids.defined() && input_ids.sizes().size() == 2, "input_ids must be a materialised [B,T] tensor");
  batch_ = input_ids.size(0);
  seq_ = input_ids.size(1);
  const int64_t tp = comm_.get_size(), rank = comm_.get_rank();
  const int64_t rows = batch_ * seq_;
  CS_ASSERT_TRUE(rows % tp == 0, "B*T (", rows, ") must be divisible by the tensor-parallel size ", tp);
  CS_ASSERT_TRUE(seq_ % (rows / tp) == 0 || (rows / tp) % seq_ == 0, "row shards must align with sequence boundaries");
  const int64_t shard = rows / tp;
  // Token and position embedding of this rank's rows only. Rows are b*T + t, so the shard is a
  // contiguous range of the flattened batch; positions repeat with period T.
  Tensor ids_shard, lab_shard;
  submit(scheduler, "cs::parallel::TPGPT2::shard_tokens", Task::Impl::kMain, Task::Impl::kCompute, {ids_shard, lab_shard},
         {input_ids, labels}, [=, T = seq_](const FnTask &) {
           // keep a [rows_in_shard / T', T'] shape so that positions line up: T' = min(T, shard)
           const int64_t cols = std::min<int64_t>(T, shard);
           ids_shard.impl()->tensor = input_ids.impl()->tensor.reshape({-1}).narrow(0, rank * shard, shard).reshape({shard / cols, cols});
           lab_shard.impl()->tensor = labels.impl()->tensor.reshape({-1}).narrow(0, rank * shard, shard).contiguous();
         });
  CS_ASSERT_TRUE(shard % seq_ == 0, "each rank must own whole sequences (B divisible by the tensor-parallel size)");
  Tensor x = compute::Embedding::forward_token_position(scheduler, wte->state(), wpe->state(), ids_shard);  // [B/tp, T, d]
  x = Utils::view(scheduler, x, {shard, config_.n_embd()});
  for (auto &block : h) x = block->forward(scheduler, x, batch_, seq_);
  x = lnf->forward(scheduler, x);
  if (!vocab_parallel_) return compute::LinearCrossEntropy::forward(scheduler, lce_state_, x, lab_shard);

  // ---- vocabulary-parallel classifier + cross-entropy ------------------------------------------------------
  // Every rank scores ALL token rows against its slice of the vocabulary; the ranks then exchange, per row, the
  // log-sum-exp over their slice and the target's logit (non-zero on the one rank that owns the target class):
  // 8 bytes per row and rank instead of a replicated classifier whose 4 * V * d byte gradient is all-reduced.
  const bool fuse = workspace_ && x.defined() && fused_tp_ok(comm_, x.impl()->tensor, rows) && scheduler.impl()->autocast_enabled;
  ce_fused_ = fuse;
  Tensor x_full;
  if (fuse) {
    x_full = lnf_full_;
    gather_rows_symmetric(scheduler, comm_, x, x_full);
  } else {
    x_full = all_gather_rows(scheduler, comm_, x);
  }
  const auto &w = lm_head->state()->forward.weight;
  const int64_t classes = w.size(0), col0 = rank * classes;
  const int64_t valid_here = std::max<int64_t>(0, std::min<int64_t>(classes, config_.vocab_size() - col0));
  Tensor logits, stats;  // [M, V/tp] local logits; [M, 2] = (lse over the local slice, target logit or 0)
  const bool amp = scheduler.impl()->autocast_enabled;
  submit(scheduler, "cs::parallel::TPGPT2::classifier_slice", Task::Impl::kMain, Task::Impl::kCompute, {logits, stats},
         {x_full, w, labels}, [=](const FnTask &task) {
           const at::Tensor &xf = x_full.impl()->tensor;
           const at::Tensor tgt = labels.impl()->tensor.reshape({-1}).contiguous();
           const int64_t M = xf.size(0);
           if (fuse) {
             const at::Tensor wc = compute::working_copy(w, at::kBFloat16);
             const int64_t n_tiles = kernels::gemm_ce_stat_tiles(classes);
             at::Tensor lg = at::empty({M, classes}, xf.options());
             at::Tensor partials = at::empty({M, n_tiles, 2}, xf.options().dtype(at::kFloat));
             at::Tensor st = at::empty({M, 2}, xf.options().dtype(at::kFloat));
             auto stream = c10::cuda::getCurrentCUDAStream().stream();
             kernels::GemmArgs g{};
             g.a = xf.data_ptr();
             g.b = wc.data_ptr();
             g.d = lg.data_ptr();
             g.stats = partials.data_ptr<float>();
             g.m = M;
             g.n = classes;
             g.k = xf.size(1);
             g.lda = g.k;
             g.ldb = g.k;
             g.ldd = classes;
             g.layout = kernels::kTN;
             g.epilogue = kernels::kEpiCrossEntropy;
             g.n_valid = std::max<int64_t>(valid_here, 1);
             const int code = kernels::gemm_bf16(stream, g);
             CS_ASSERT_TRUE(code == 0, "classifier slice GEMM launch failed (", code, ")");
             task.intermediate().push_back(partials);
             const int rc = kernels::cross_entropy_slice_stats(stream, partials.data_ptr<float>(), n_tiles, lg.data_ptr(), classes,
                                                               tgt.data_ptr<int64_t>(), col0, valid_here, st.data_ptr<float>(), M);
             CS_ASSERT_TRUE(rc == 0, "cross_entropy_slice_stats failed: ", cuda_error_string(rc));
             logits.impl()->tensor = lg;
             stats.impl()->tensor = st;
             return;
           }
           const at::ScalarType ct = xf.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
           const at::ScalarType dt = amp && xf.is_cuda() ? at::kBFloat16 : xf.scalar_type();
           at::Tensor lg = at::linear(xf.to(dt), compute::working_copy(w, dt));
           at::Tensor lf = lg.to(ct);
           if (valid_here < classes) lf = lf.clone(), lf.narrow(1, valid_here, classes - valid_here).fill_(-INFINITY);
           at::Tensor lse = valid_here > 0 ? at::logsumexp(lf, {1}) : at::full({M}, -INFINITY, lf.options());
           at::Tensor local = tgt - col0;
           at::Tensor mine = local.ge(0).logical_and(local.lt(valid_here));
           at::Tensor picked = lg.to(ct).gather(1, at::where(mine, local, at::zeros_like(local)).unsqueeze(1)).squeeze(1);
           logits.impl()->tensor = lg;
           stats.impl()->tensor = at::stack({lse, at::where(mine, picked, at::zeros_like(picked))}, 1).contiguous();
         });
  Tensor all_stats;  // [tp * M, 2]
  if (fuse) {
    all_stats = stats_full_;
    gather_rows_symmetric(scheduler, comm_, stats, all_stats);
  } else {
    all_stats = all_gather_rows(scheduler, comm_, stats);
  }
  Tensor loss, lse;  // lse: [M + 1] = global log-sum-exp per row, then the number of rows that count
  submit(scheduler, "cs::parallel::TPGPT2::combine_loss", Task::Impl::kMain, Task::Impl::kCompute, {loss, lse}, {all_stats, labels},
         [=](const FnTask &) {
           const at::Tensor tgt = labels.impl()->tensor.reshape({-1});
           const int64_t M = tgt.numel();
           const at::Tensor st = all_stats.impl()->tensor.view({tp, M, 2});
           at::Tensor global = at::logsumexp(st.select(2, 0), {0});
           at::Tensor target_logit = st.select(2, 1).sum(0);
           at::Tensor keep = tgt.ne(-100).to(st.scalar_type());
           at::Tensor count = keep.sum().clamp_min(1.0);
           loss.impl()->tensor = ((global - target_logit) * keep).sum() / count;
           lse.impl()->tensor = at::cat({global, count.reshape({1})}).contiguous();
         });
  ce_logits_ = logits;
  ce_lse_ = lse;
  ce_labels_ = labels;
  ce_input_ = x_full;
  return loss;
}

void TPGPT2Impl::backward_loss(const Scheduler &scheduler, const models::GradientSync &sync) {
  namespace Utils = compute::Utils;
  Tensor grad;
  if (!vocab_parallel_) {
    grad = compute::LinearCrossEntropy::backward(scheduler, lce_state_);
    sync.push(scheduler, lm_head->state()->forward.grad_weight);
  } else {
    const int64_t tp = comm_.get_size(), rank = comm_.get_rank();
    const auto &w = lm_head->state()->forward.weight;
    const int64_t classes = w.size(0), col0 = rank * classes;
    const int64_t valid_here = std::max<int64_t>(0, std::min<int64_t>(classes, config_.vocab_size() - col0));
    Tensor dlogits;
    // logits -> (softmax - onehot) * tp / count, in place on the GPU path. The factor tp keeps the convention of the
    // data-parallel trainer: the optimizer multiplies every gradient by 1 / world.
    submit(scheduler, "cs::parallel::TPGPT2::classifier_slice_backward", Task::Impl::kMain, Task::Impl::kCompute, {dlogits},
           {ce_logits_, ce_lse_, ce_labels_}, [=, lg_h = ce_logits_, lse_h = ce_lse_, lab = ce_labels_, fuse = ce_fused_](const FnTask &) {
             at::Tensor lg = lg_h.impl()->tensor;
             const at::Tensor &ls = lse_h.impl()->tensor;
             const at::Tensor tgt = lab.impl()->tensor.reshape({-1}).contiguous();
             const int64_t M = lg.size(0);
             if (fuse) {
               const int rc = kernels::cross_entropy_backward_inplace(c10::cuda::getCurrentCUDAStream().stream(), lg.data_ptr(), classes,
                                                                      ls.data_ptr<float>(), tgt.data_ptr<int64_t>(), ls.data_ptr<float>() + M,
                                                                      static_cast<float>(tp), M, classes, col0 + valid_here, -100, col0);
               CS_ASSERT_TRUE(rc == 0, "cross_entropy_backward_inplace failed: ", cuda_error_string(rc));
               dlogits.impl()->tensor = lg;
               return;
             }
             const at::ScalarType ct = lg.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
             at::Tensor p = at::exp(lg.to(ct) - ls.narrow(0, 0, M).to(ct).unsqueeze(1));
             if (valid_here < classes) p.narrow(1, valid_here, classes - valid_here).zero_();
             at::Tensor keep = tgt.ne(-100);
             at::Tensor local = tgt - col0;
             at::Tensor mine = local.ge(0).logical_and(local.lt(valid_here)).logical_and(keep);
             p.scatter_add_(1, at::where(mine, local, at::zeros_like(local)).unsqueeze(1), -mine.to(ct).unsqueeze(1));
             p.mul_(keep.to(ct).unsqueeze(1));
             p.mul_(static_cast<double>(tp)).div_(ls.narrow(0, M, 1).to(ct));
             dlogits.impl()->tensor = p.to(lg.scalar_type());
           });
    auto st = lm_head->state();
    st->backward.input = ce_input_;
    if (ce_fused_) {
      st->forward.weight.impl()->autocast_enabled = true;
      st->forward.weight.impl()->autocast_dtype = at::kBFloat16;
      grad = (batch_ * seq_ / tp) % 256 == 0 ? gemm_scatter(scheduler, comm_, w, dlogits, nullptr, true, *workspace_)
                                             : row_parallel_symmetric(scheduler, comm_, w, dlogits, nullptr, true, workspace_->partial);
    } else {
      grad = reduce_scatter_rows(scheduler, comm_, lm_head->backward_input(scheduler, dlogits));
    }
    lm_head->backward_parameter(scheduler, dlogits);
    ce_logits_ = Tensor{};
    ce_lse_ = Tensor{};
    ce_labels_ = ReadOnlyTensor{};
    ce_input_ = Tensor{};
  }
  grad = lnf->backward(scheduler, grad);
  sync.push(scheduler, lnf->state()->forward.grad_weight);
  sync.push(scheduler, lnf->state()->forward.grad_bias);
  for (auto it = h.rbegin(); it != h.rend(); ++it) grad = (*it)->backward(scheduler, grad, sync);
  const int64_t shard = batch_ * seq_ / comm_.get_size();
  grad = Utils::view(scheduler, grad, {shard / seq_, seq_, config_.n_embd()});
  compute::Embedding::backward_token_position(scheduler, wte->state(), wpe->state(), grad);
  sync.push(scheduler, wpe->state()->forward.grad_weight);
  sync.push(scheduler, wte->state()->forward.grad_weight);
}
}  // namespace cs::parallel
