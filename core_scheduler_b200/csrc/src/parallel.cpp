// ZeRO-style sharded optimizer and symmetric-memory flattening. See cs/parallel.h.
#include "cs/parallel.h"

#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <cmath>
#include <unordered_map>

#include "kernels/collectives.h"
#include "symm_internal.h"

namespace cs::parallel {
using communication::SymmetricContext;

std::shared_ptr<module::FlatParameters> flatten_symmetric(const Scheduler &scheduler, const module::Module &module,
                                                         const communication::Comm &comm, optional<at::ScalarType> lp_dtype) {
  auto ctx = comm.impl()->symmetric;
  module::FlattenOptions opts;
  opts.lp_dtype(lp_dtype).transposed_copies(false).pad_total_to(comm.get_size() * 128);
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
             const kernels::PeerTable table = communication::table_of(*ctx);
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
             // one launch: "every rank's gradients are complete" and "every rank's bf16 arena received all
             // shards" are the barriers at the two ends of the kernel
             int blocks = 0;
             const auto h = communication::begin_collective(*ctx, kernels::kChanZero);
             const int code = kernels::symm_reduce_scatter_adamw_all_gather(c10::cuda::getCurrentCUDAStream().stream(), table, h, a, &blocks);
             CS_ASSERT_TRUE(code == 0, "fused reduce-scatter/AdamW/all-gather launch failed: ", cuda_error_string(code));
             communication::end_collective(*ctx, kernels::kChanZero, blocks);
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

// ------------------------------------------------------------ fused TP GEMM + collective ----
namespace {
std::atomic<int64_t> g_fused_tp_launches{0};

struct SymmetricSlots {
  communication::SymmetricBlock block[2];
  int next{0};
};
// Per-context staging buffers for the fused paths (allocated on first use, identical call
// sequences on every rank give identical offsets).
std::unordered_map<const communication::SymmetricContext *, SymmetricSlots> g_ag_slots, g_rs_slots;

communication::SymmetricBlock next_slot(std::unordered_map<const communication::SymmetricContext *, SymmetricSlots> &table,
                                        communication::SymmetricContext &ctx, int64_t bytes, bool alternate) {
  auto &slots = table[&ctx];
  const int idx = alternate ? slots.next : 0;
  if (alternate) slots.next ^= 1;
  if (slots.block[idx].bytes < bytes) {
    if (slots.block[idx].bytes > 0) ctx.release(slots.block[idx]);
    slots.block[idx] = ctx.allocate(bytes);
  }
  return slots.block[idx];
}

bool fused_tp_ok(const communication::Comm &comm, const at::Tensor &x, int64_t total_rows) {
  auto ctx = comm.impl()->symmetric;
  const int64_t tp = comm.get_size();
  return ctx && tp > 1 && tp <= 8 && x.is_cuda() && x.scalar_type() == at::kBFloat16 &&
         compute::get_backend() == compute::Backend::kFused && total_rows % tp == 0 && (total_rows / tp) % 256 == 0 &&
         std::getenv("CS_TP_UNFUSED") == nullptr;
}
}  // namespace

int64_t fused_tp_launches() { return g_fused_tp_launches.load(); }

Tensor column_parallel_forward(const Scheduler &scheduler, const communication::Comm &comm,
                               const std::shared_ptr<compute::Linear::State> &state, const ReadOnlyTensor &x_shard) {
  const int64_t tp = comm.get_size();
  // The fused kernel fetches the other ranks' rows by TMA straight from peer memory, once per output-column tile
  // (peer data is not cached in the local L2): for wide layers that is several times the bytes of one
  // all-gather. CS_TP_FUSED_ALL_GATHER=1 selects it; the default gathers the rows once with the peer-copy kernel
  // and runs the GEMM on local memory.
  static const bool fused_gather = std::getenv("CS_TP_FUSED_ALL_GATHER") != nullptr;
  const bool can_fuse = fused_gather && x_shard.defined() && fused_tp_ok(comm, x_shard.impl()->tensor, x_shard.size(0) * tp) &&
                        scheduler.impl()->autocast_enabled && !state->args.bias;
  if (!can_fuse) {
    Tensor full = all_gather_rows(scheduler, comm, x_shard);
    return compute::Linear::forward(scheduler, state, full);
  }
  Tensor out;
  const bool gelu = state->args.gelu_epilogue;
  state->backward.input = Tensor{};  // backward re-gathers the input; nothing is kept alive here
  state->forward.weight.impl()->autocast_enabled = true;
  state->forward.weight.impl()->autocast_dtype = at::kBFloat16;
  submit(scheduler, "cs::parallel::column_parallel_forward(all-gather+GEMM)", Task::Impl::kMain, Task::Impl::kCompute, {out},
         {x_shard, state->forward.weight}, [out, x_shard, w = state->forward.weight, comm, gelu, tp](const FnTask &) {
           auto &ctx = *comm.impl()->symmetric;
           const at::Tensor xs = x_shard.impl()->tensor.contiguous();
           const at::Tensor wc = compute::working_copy(w, at::kBFloat16);
           const int64_t rows = xs.size(0), k = xs.size(1), n = wc.size(0);
           const auto slot = next_slot(g_ag_slots, ctx, rows * k * 2, true);
           auto stream = c10::cuda::getCurrentCUDAStream().stream();
           CS_CHECK_CUDART(cudaMemcpyAsync(ctx.bases[ctx.rank] + slot.offset, xs.data_ptr(), static_cast<size_t>(rows * k * 2),
                                           cudaMemcpyDeviceToDevice, stream));
           ctx.barrier();  // every rank's shard is in place (and the slot's previous readers are done)
           at::Tensor y = at::empty({rows * tp, n}, xs.options());
           at::Tensor y2;
           kernels::GemmArgs g{};
           g.b = wc.data_ptr();
           g.d = y.data_ptr();
           g.m = rows * tp;
           g.n = n;
           g.k = k;
           g.lda = k;
           g.ldb = k;
           g.ldd = n;
           g.layout = kernels::kTN;
           g.epilogue = kernels::kEpiStoreBf16;
           if (gelu) {
             y2 = at::empty_like(y);
             g.d2 = y2.data_ptr();
             g.epilogue = kernels::kEpiGeluDual;
           }
           g.peer_count = static_cast<int>(tp);
           g.peer_rank = ctx.rank;
           for (int p = 0; p < tp; ++p) g.a_peers[p] = ctx.bases[p] + slot.offset;
           const int code = kernels::gemm_bf16(stream, g);
           CS_ASSERT_TRUE(code == 0, "fused all-gather+GEMM launch failed (", code, ")");
           g_fused_tp_launches.fetch_add(1);
           out.impl()->tensor = y;
           out.impl()->companion = y2;
         });
  return out;
}

Tensor row_parallel_forward(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &weight,
                            const ReadOnlyTensor &x, const ReadOnlyTensor *residual_shard, bool weight_is_rhs) {
  // weight_is_rhs == false: y = x * W^T with W [out, in_local]      (forward of c_proj / fc2)
  // weight_is_rhs == true : y = x * W   with W [out_local, in]      (input gradient of c_attn / fc1)
  const int64_t tp = comm.get_size();
  Tensor out;
  std::vector<ReadOnlyTensor> ins{x, weight};
  std::optional<ReadOnlyTensor> res;
  if (residual_shard) {
    res = *residual_shard;
    ins.push_back(*residual_shard);
  }
  submit(scheduler, "cs::parallel::row_parallel_forward(GEMM+reduce-scatter)", Task::Impl::kMain, Task::Impl::kCompute, {out}, ins,
         [out, x, weight, res, comm, tp, weight_is_rhs](const FnTask &) {
           auto &ctx = *comm.impl()->symmetric;
           const at::Tensor xa = x.impl()->tensor.reshape({-1, x.impl()->tensor.size(-1)}).contiguous();
           const at::Tensor wc = compute::working_copy(weight, at::kBFloat16);
           const int64_t m = xa.size(0), k = xa.size(1);
           const int64_t n = weight_is_rhs ? wc.size(1) : wc.size(0);
           const int64_t rows = m / tp;
           const auto slot = next_slot(g_rs_slots, ctx, rows * n * 4, false);
           auto stream = c10::cuda::getCurrentCUDAStream().stream();
           float *acc = reinterpret_cast<float *>(ctx.bases[ctx.rank] + slot.offset);
           CS_CHECK_CUDART(cudaMemsetAsync(acc, 0, static_cast<size_t>(rows * n * 4), stream));
           ctx.barrier();  // all accumulators are zero before anybody adds
           kernels::GemmArgs g{};
           g.a = xa.data_ptr();
           g.b = wc.data_ptr();
           g.m = m;
           g.n = n;
           g.k = k;
           g.lda = k;
           g.ldb = weight_is_rhs ? n : k;
           g.ldd = n;
           g.layout = weight_is_rhs ? kernels::kTM : kernels::kTN;
           g.epilogue = kernels::kEpiAccumF32;
           g.peer_count = static_cast<int>(tp);
           g.peer_rank = ctx.rank;
           for (int p = 0; p < tp; ++p) g.d_peers[p] = ctx.bases[p] + slot.offset;
           const int code = kernels::gemm_bf16(stream, g);
           CS_ASSERT_TRUE(code == 0, "fused GEMM+reduce-scatter launch failed (", code, ")");
           g_fused_tp_launches.fetch_add(1);
           ctx.barrier();  // every rank's tiles have been added into our rows
           at::Tensor y = at::empty({rows, n}, xa.options());
           at::Tensor r;
           if (res) r = res->impl()->tensor.contiguous();
           const int rc = kernels::add_f32_residual_to_bf16(stream, acc, res ? r.data_ptr() : nullptr, y.data_ptr(), rows * n);
           CS_ASSERT_TRUE(rc == 0, "accumulator finalisation failed");
           out.impl()->tensor = y;
         });
  return out;
}

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
  const bool fuse = x_shard.defined() && fused_tp_ok(comm, x_shard.impl()->tensor, batch * seq) &&
                    scheduler.impl()->autocast_enabled;
  saved_ln1_out = Tensor{};
  saved_ln2_out = Tensor{};
  Tensor a = ln1->forward(scheduler, x_shard);                 // [M/tp, d]
  Tensor qkv;                                                   // [M, 3 d/tp]
  if (fuse) {
    saved_ln1_out = a;  // backward re-gathers it for the weight gradient
    qkv = column_parallel_forward(scheduler, comm, c_attn->state(), a);
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
    x1 = row_parallel_forward(scheduler, comm, c_proj->state()->forward.weight, ctx2, &x_shard, false);
  } else {
    x1 = reduce_scatter_rows(scheduler, comm, c_proj->forward(scheduler, ctx2), &x_shard);
  }
  Tensor b = ln2->forward(scheduler, x1);
  Tensor pre;                                                    // [M, 4d/tp], carries GELU
  if (fuse) {
    saved_ln2_out = b;
    pre = column_parallel_forward(scheduler, comm, fc1->state(), b);
  } else {
    pre = fc1->forward(scheduler, all_gather_rows(scheduler, comm, b));
  }
  if (!fuse) return reduce_scatter_rows(scheduler, comm, fc2->forward(scheduler, pre), &x1);
  // fused fc2: GELU(pre) is the companion emitted by the fc1 epilogue
  Tensor act;
  submit(scheduler, "cs::parallel::TPBlock::activation_view", Task::Impl::kMain, Task::Impl::kCompute, {act}, {pre},
         [act, pre](const FnTask &) { act.impl()->tensor = pre.impl()->companion; });
  auto fs = fc2->state();
  fs->backward.input = pre;
  fs->backward.activated = act;
  fs->backward.input_count = 2;
  fs->forward.weight.impl()->autocast_enabled = true;
  fs->forward.weight.impl()->autocast_dtype = at::kBFloat16;
  return row_parallel_forward(scheduler, comm, fs->forward.weight, act, &x1, false);
}

Tensor TPBlockImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_shard, const models::GradientSync &sync) {
  namespace Utils = compute::Utils;
  // MLP: reduce-scatter backward = all-gather of the incoming row shard
  Tensor dz = all_gather_rows(scheduler, comm, grad_shard);      // [M, d]
  Tensor d_pre = fc2->backward_input(scheduler, dz);
  fc2->backward_parameter(scheduler, dz);
  const bool fused_bwd = saved_ln2_out.defined();
  Tensor d_b;                                                    // all-gather backward = reduce-scatter
  if (fused_bwd) {
    d_b = row_parallel_forward(scheduler, comm, fc1->state()->forward.weight, d_pre, nullptr, true);
    fc1->state()->backward.input = all_gather_rows(scheduler, comm, saved_ln2_out);  // re-gather for the weight gradient
  } else {
    d_b = reduce_scatter_rows(scheduler, comm, fc1->backward_input(scheduler, d_pre));
  }
  fc1->backward_parameter(scheduler, d_pre);
  Tensor d_x1 = ln2->backward(scheduler, d_b, grad_shard);       // + residual branch
  sync.push(scheduler, ln2->state()->forward.grad_weight);
  sync.push(scheduler, ln2->state()->forward.grad_bias);
  // attention
  Tensor dy = all_gather_rows(scheduler, comm, d_x1);
  Tensor d_ctx = c_proj->backward_input(scheduler, dy);          // [M, d/tp]
  c_proj->backward_parameter(scheduler, dy);
  Tensor d_qkv = compute::ScaledDotProductAttention::backward_packed(scheduler, attn_state, d_ctx);
  const int64_t three_d_local = c_attn->state()->forward.weight.size(0);
  Tensor d_qkv2 = Utils::view(scheduler, d_qkv, {-1, three_d_local});
  Tensor d_a;
  if (fused_bwd) {
    d_a = row_parallel_forward(scheduler, comm, c_attn->state()->forward.weight, d_qkv2, nullptr, true);
    c_attn->state()->backward.input = all_gather_rows(scheduler, comm, saved_ln1_out);
  } else {
    d_a = reduce_scatter_rows(scheduler, comm, c_attn->backward_input(scheduler, d_qkv2));
  }
  c_attn->backward_parameter(scheduler, d_qkv2);
  saved_ln1_out = Tensor{};
  saved_ln2_out = Tensor{};
  Tensor d_x = ln1->backward(scheduler, d_a, d_x1);
  sync.push(scheduler, ln1->state()->forward.grad_weight);
  sync.push(scheduler, ln1->state()->forward.grad_bias);
  return d_x;
}

TPGPT2Impl::TPGPT2Impl(const Scheduler &scheduler, const models::GPT2Config &config, const communication::Comm &comm)
    : config_{config}, comm_{comm} {
  const auto dev = config.device().value_or(scheduler.device());
  const int64_t d = config.n_embd();
  wte = register_module("wte", module::Embedding{scheduler, compute::Embedding::Options{config.padded_vocab_size(), d}.device(dev).dtype(config.dtype())});
  wpe = register_module("wpe", module::Embedding{scheduler, compute::Embedding::Options{config.block_size(), d}.device(dev).dtype(config.dtype())});
  compute::Utils::normal_(scheduler, wte->state()->forward.weight, 0, config.init_std());
  compute::Utils::normal_(scheduler, wpe->state()->forward.weight, 0, config.init_std());
  for (int64_t l = 0; l < config.n_layer(); ++l) h.push_back(register_module(std::to_string(l), TPBlock{scheduler, config, comm}));
  lnf = register_module("lnf", module::LayerNorm{scheduler, compute::LayerNorm::Options{d}.device(dev).dtype(config.dtype())});
  lm_head = register_module("lm_head", module::Linear{scheduler, compute::Linear::Options{d, config.padded_vocab_size()}.bias(false).device(dev).dtype(config.dtype())});
  compute::Utils::normal_(scheduler, lm_head->state()->forward.weight, 0, config.init_std());
  lce_state_ = compute::LinearCrossEntropy::init(scheduler, lm_head->state(), config.vocab_size(), -100);
}

std::vector<std::string> TPGPT2Impl::replicated_parameters() const {
  std::vector<std::string> out{"wte.weight", "wpe.weight", "lnf.weight", "lnf.bias", "lm_head.weight"};
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
  return compute::LinearCrossEntropy::forward(scheduler, lce_state_, x, lab_shard);
}

void TPGPT2Impl::backward_loss(const Scheduler &scheduler, const models::GradientSync &sync) {
  namespace Utils = compute::Utils;
  Tensor grad = compute::LinearCrossEntropy::backward(scheduler, lce_state_);
  sync.push(scheduler, lm_head->state()->forward.grad_weight);
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
