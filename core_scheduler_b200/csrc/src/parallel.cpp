// ZeRO-style sharded optimizer and symmetric-memory flattening. See cs/parallel.h.
#include "cs/parallel.h"

#include <c10/cuda/CUDAStream.h>

#include <cmath>

#include "kernels/collectives.h"

namespace cs::parallel {
using communication::SymmetricContext;

std::shared_ptr<module::FlatParameters> flatten_symmetric(const Scheduler &scheduler, const module::Module &module,
                                                         const communication::Comm &comm, optional<at::ScalarType> lp_dtype) {
  auto ctx = comm.impl()->symmetric;
  module::FlattenOptions opts;
  opts.lp_dtype(lp_dtype).transposed_copies(true).pad_total_to(comm.get_size() * 128);
  if (ctx) {
    opts.arena_allocator([ctx](int64_t bytes) {
      const auto block = ctx->allocate(bytes);
      return ctx->tensor(block, {bytes}, at::kByte);
    });
  }
  return module::flatten_parameters(scheduler, module, opts);
}

ZeroAdamWImpl::ZeroAdamWImpl(const Scheduler &scheduler, const module::Module &module,
                             const std::shared_ptr<module::FlatParameters> &flat, const communication::Comm &comm,
                             const Options &options)
    : flat_{flat}, comm_{comm} {
  bind(&module);
  flat->params.wait();
  CS_ASSERT_TRUE(flat->params.impl()->tensor.scalar_type() == at::kFloat, "ZeroAdamW needs fp32 master parameters");
  const int64_t world = comm.get_size();
  CS_ASSERT_TRUE(flat->total % (world * 4) == 0, "arena length must split into 4-element aligned shards");
  shard_count_ = flat->total / world;
  shard_begin_ = shard_count_ * comm.get_rank();
  // moments only for this rank's shard
  Tensor shard;
  submit(scheduler, "cs::parallel::ZeroAdamW::shard_view", Task::Impl::kMain, Task::Impl::kCompute, {shard}, {flat->params},
         [shard, flat, b = shard_begin_, n = shard_count_](const FnTask &) {
           shard.impl()->tensor = flat->params.impl()->tensor.narrow(0, b, n);
         });
  state_ = optimizer::AdamW::init(scheduler, shard, options);
  states_.insert("__shard__", state_);
}

OrderedDict<std::string, Tensor> ZeroAdamWImpl::named_state_tensors() const {
  OrderedDict<std::string, Tensor> out;
  out.insert(str_cat("shard", comm_.get_rank(), ".m"), state_->tensors.m);
  out.insert(str_cat("shard", comm_.get_rank(), ".v"), state_->tensors.v);
  return out;
}

void ZeroAdamWImpl::step(const Scheduler &scheduler) {
  const module::Module *m = model();
  CS_ASSERT_TRUE(m != nullptr, "the optimised module is gone");
  auto ctx = comm_.impl()->symmetric;
  const int64_t t = ++state_->options.t;
  auto named = m->named_parameters();
  std::vector<Tensor> touched;
  for (auto &slot : flat_->slots) touched.push_back(named[slot.key]);
  {
    std::vector<ReadOnlyTensor> writers(flat_->grad_handles.begin(), flat_->grad_handles.end());
    submit(scheduler, "cs::parallel::ZeroAdamW::join_gradients", Task::Impl::kComm, Task::Impl::kCompute, {flat_->grads}, writers,
           [handles = flat_->grad_handles](const FnTask &) {
             for (auto &h : handles)
               if (h.impl()->fresh && h.impl()->tensor.defined()) h.impl()->tensor.zero_();
           });
  }
  std::vector<Tensor> outs{flat_->params, flat_->lp, state_->tensors.m, state_->tensors.v};
  outs.insert(outs.end(), touched.begin(), touched.end());
  submit(scheduler, "cs::parallel::ZeroAdamW::step", Task::Impl::kComm, Task::Impl::kNccl, outs, {flat_->grads},
         [flat = flat_, state = state_, ctx, t, b = shard_begin_, n = shard_count_, world = comm_.get_size(),
          touched](const FnTask &) {
           const auto &o = state->options;
           const double bc1 = 1.0 - std::pow(o.beta1, static_cast<double>(t));
           const double bc2 = 1.0 - std::pow(o.beta2, static_cast<double>(t));
           at::Tensor &P = flat->params.impl()->tensor;
           at::Tensor &G = flat->grads.impl()->tensor;
           at::Tensor &L = flat->lp.impl()->tensor;
           if (ctx && P.is_cuda()) {
             int64_t g_off = 0, l_off = -1;
             CS_ASSERT_TRUE(ctx->locate(G.data_ptr(), static_cast<int64_t>(G.nbytes()), &g_off),
                            "ZeroAdamW needs the gradient arena in symmetric memory (use flatten_symmetric)");
             if (L.defined())
               CS_ASSERT_TRUE(ctx->locate(L.data_ptr(), static_cast<int64_t>(L.nbytes()), &l_off),
                              "ZeroAdamW needs the bf16 arena in symmetric memory (use flatten_symmetric)");
             kernels::PeerTable table{};
             for (int p = 0; p < ctx->size; ++p) {
               table.base[p] = ctx->bases[p];
               table.flags[p] = ctx->flags[p];
             }
             table.rank = ctx->rank;
             table.size = ctx->size;
             kernels::ShardedAdamWArgs a{};
             a.grad_offset_bytes = g_off;
             a.lp_offset_bytes = l_off;
             a.master = P.data_ptr<float>() + b;
             a.exp_avg = state->tensors.m.impl()->tensor.data_ptr<float>();
             a.exp_avg_sq = state->tensors.v.impl()->tensor.data_ptr<float>();
             a.shard_begin = b;
             a.shard_count = n;
             a.lr = static_cast<float>(o.lr);
             a.beta1 = static_cast<float>(o.beta1);
             a.beta2 = static_cast<float>(o.beta2);
             a.eps = static_cast<float>(o.eps);
             a.weight_decay = static_cast<float>(o.weight_decay);
             a.inv_bias_correction1 = static_cast<float>(1.0 / bc1);
             a.inv_bias_correction2 = static_cast<float>(1.0 / bc2);
             a.grad_scale = static_cast<float>(o.grad_scale / static_cast<double>(world));
             a.clip_coef = state->clip_coef.impl()->tensor.defined() ? state->clip_coef.impl()->tensor.data_ptr<float>() : nullptr;
             ctx->barrier();  // every rank's gradients are complete
             const int code = kernels::symm_reduce_scatter_adamw_all_gather(c10::cuda::getCurrentCUDAStream().stream(), table, a);
             CS_ASSERT_TRUE(code == 0, "fused reduce-scatter/AdamW/all-gather launch failed: ", cuda_error_string(code));
             ctx->barrier();  // every rank's bf16 arena received all shards
           } else {
             // Single rank (or CPU): plain sharded update on the whole arena.
             CS_ASSERT_TRUE(world == 1, "ZeroAdamW across ranks needs symmetric memory on CUDA devices");
             at::Tensor g = G.to(at::kFloat) * o.grad_scale;
             at::Tensor w = P, mm = state->tensors.m.impl()->tensor, vv = state->tensors.v.impl()->tensor;
             w.mul_(1 - o.lr * o.weight_decay);
             mm.mul_(o.beta1).add_(g, 1 - o.beta1);
             vv.mul_(o.beta2).addcmul_(g, g, 1 - o.beta2);
             w.sub_((mm / bc1) / ((vv / bc2).sqrt() + o.eps) * o.lr);
             if (L.defined()) L.copy_(w);
           }
           for (auto &p : touched) {
             auto &impl = *p.impl();
             ++impl.version;
             if (impl.lp.defined()) impl.lp_version = impl.version;
             if (impl.lp_t.defined()) {
               // the transpose is rebuilt from the fresh bf16 copy (the fp32 arena is only
               // authoritative inside this rank's shard)
               impl.lp_t.copy_(impl.lp.t());
               impl.lp_t_version = impl.version;
             }
           }
         });
}

void ZeroAdamWImpl::gather_master(const Scheduler &scheduler) {
  const int64_t world = comm_.get_size();
  if (world <= 1) return;
  std::vector<Tensor> recv(static_cast<size_t>(world));
  Tensor send;
  std::vector<Tensor> outs = recv;
  outs.push_back(send);
  submit(scheduler, "cs::parallel::ZeroAdamW::shard_views", Task::Impl::kMain, Task::Impl::kCompute, outs, {flat_->params},
         [flat = flat_, recv, send, n = shard_count_, b = shard_begin_](const FnTask &) {
           const at::Tensor &P = flat->params.impl()->tensor;
           for (size_t r = 0; r < recv.size(); ++r) recv[r].impl()->tensor = P.narrow(0, static_cast<int64_t>(r) * n, n);
           send.impl()->tensor = P.narrow(0, b, n).clone();
         });
  communication::AllGather::run(scheduler, comm_, {recv}, {send});
}
}  // namespace cs::parallel
