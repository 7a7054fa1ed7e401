// SPDX-License-Identifier: Apache-2.0
// ScaledDotProductAttention, Utils and Init. See cs/compute.h.
// Reference behaviour studied in src/compute/{sdpa_flash_attn,sdpa_cudnn,utils,init}.cpp of the
// reference project: q/k/v arrive as [B,T,H,D]; backward returns dq,dk,dv in the same layout;
// Utils wraps tensor factories/views as scheduler tasks; clip_grad_norm_ scales in place by
// min(1, max_norm/(norm+1e-6)).
#include <ATen/cuda/CUDAContext.h>

#include <cmath>
#include <cstdlib>
#include <limits>
#include <string>

#include "cs/compute.h"
#include "op_common.h"

namespace cs::compute {
using namespace detail;

std::shared_ptr<ScaledDotProductAttention::State> ScaledDotProductAttention::init(const Scheduler &,
                                                                                  const Options &options) {
  auto state = std::make_shared<State>();
  state->args = State::Args{options.dropout_p(), options.is_causal(), options.return_debug_mask(), options.scale()};
  return state;
}

namespace {
struct SdpaOut {
  at::Tensor out, lse;
};

// Reference math in fp32/fp64 on [B,H,T,D] views; keeps only the row log-sum-exp.
SdpaOut sdpa_math_forward(const at::Tensor &q, const at::Tensor &k, const at::Tensor &v, bool causal, double scale) {
  const at::ScalarType ct = q.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
  at::Tensor s = at::matmul(q.to(ct), k.to(ct).transpose(-1, -2)).mul_(scale);
  if (causal) {
    const int64_t Tq = q.size(-2), Tk = k.size(-2);
    at::Tensor mask = at::ones({Tq, Tk}, q.options().dtype(at::kBool)).tril_(Tk - Tq);
    s.masked_fill_(mask.logical_not(), -std::numeric_limits<double>::infinity());
  }
  at::Tensor lse = at::logsumexp(s, {-1});
  at::Tensor p = at::exp(s - lse.unsqueeze(-1));
  return {at::matmul(p, v.to(ct)).to(q.scalar_type()), lse};
}

std::array<at::Tensor, 3> sdpa_math_backward(const at::Tensor &dout, const at::Tensor &q, const at::Tensor &k,
                                             const at::Tensor &v, const at::Tensor &out, const at::Tensor &lse,
                                             bool causal, double scale) {
  const at::ScalarType ct = q.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
  const at::Tensor qf = q.to(ct), kf = k.to(ct), vf = v.to(ct), dof = dout.to(ct), of = out.to(ct);
  at::Tensor s = at::matmul(qf, kf.transpose(-1, -2)).mul_(scale);
  if (causal) {
    const int64_t Tq = q.size(-2), Tk = k.size(-2);
    at::Tensor mask = at::ones({Tq, Tk}, q.options().dtype(at::kBool)).tril_(Tk - Tq);
    s.masked_fill_(mask.logical_not(), -std::numeric_limits<double>::infinity());
  }
  at::Tensor p = at::exp(s - lse.to(ct).unsqueeze(-1));
  at::Tensor dv = at::matmul(p.transpose(-1, -2), dof);
  at::Tensor dp = at::matmul(dof, vf.transpose(-1, -2));
  at::Tensor delta = at::sum(dof * of, {-1}, true);
  at::Tensor ds = p * (dp - delta);
  at::Tensor dq = at::matmul(ds, kf).mul_(scale);
  at::Tensor dk = at::matmul(ds.transpose(-1, -2), qf).mul_(scale);
  return {dq.to(q.scalar_type()), dk.to(q.scalar_type()), dv.to(q.scalar_type())};
}

bool library_flash_ok(const at::Tensor &q) {
  return q.is_cuda() && (q.scalar_type() == at::kHalf || q.scalar_type() == at::kBFloat16) && q.size(-1) % 8 == 0 &&
         q.size(-1) <= 256;
}

// Library engine for half/bf16 CUDA attention: "cudnn" (fused flash attention of cuDNN, the
// counterpart of the reference's ScaledDotProductCuDnn) or "flash" (the flash-attention kernels
// bundled with libtorch, the counterpart of ScaledDotProductFlashAttention).
bool use_cudnn_engine() {
  static const bool cudnn = [] {
    const char *e = std::getenv("CS_ATTENTION_ENGINE");
    return e == nullptr || std::string(e) != "flash";
  }();
  return cudnn;
}

// This library's own forward and backward kernels on the packed qkv tensor are the default for
// the shapes they cover (bf16, causal, head dimension 64, T % 128 == 0, no dropout);
// CS_ATTENTION_ENGINE=cudnn or =flash selects a library engine instead. Read at every call (a
// dozen per step) so that a process can switch engines between models.
bool use_own_forward() {
  const char *e = std::getenv("CS_ATTENTION_ENGINE");
  return e == nullptr || std::string(e) == "tcgen05";
}

double resolve_scale(const optional<double> &scale, int64_t head_dim) {
  return scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(head_dim));
}

struct Saved {
  Tensor out, lse, cum_q, cum_k, seed, offset;
};

// q,k,v: [B,T,H,D] tensors (any strides). Fills `saved` and returns out [B,T,H,D].
at::Tensor attention_forward_body(const at::Tensor &q4, const at::Tensor &k4, const at::Tensor &v4,
                                  const ScaledDotProductAttention::State::Args &args,
                                  ScaledDotProductAttention::State::Backward *bw_meta, const Saved &saved) {
  const at::Tensor q = q4.transpose(1, 2), k = k4.transpose(1, 2), v = v4.transpose(1, 2);  // [B,H,T,D]
  const double scale = resolve_scale(args.scale, q.size(-1));
  if (library_flash_ok(q) && use_cudnn_engine() && q.size(-1) <= 128) {
    auto r = at::_scaled_dot_product_cudnn_attention(q, k, v, std::nullopt, true, args.dropout_p, args.is_causal,
                                                     args.return_debug_mask, scale);
    saved.out.impl()->tensor = std::get<0>(r);
    saved.lse.impl()->tensor = std::get<1>(r);
    saved.cum_q.impl()->tensor = std::get<2>(r);
    saved.cum_k.impl()->tensor = std::get<3>(r);
    bw_meta->max_q = std::get<4>(r).expect_int();
    bw_meta->max_k = std::get<5>(r).expect_int();
    saved.seed.impl()->tensor = std::get<6>(r);
    saved.offset.impl()->tensor = std::get<7>(r);
    return std::get<0>(r).transpose(1, 2);
  }
  if (library_flash_ok(q)) {
    auto r = at::_scaled_dot_product_flash_attention(q, k, v, args.dropout_p, args.is_causal, args.return_debug_mask,
                                                     scale);
    saved.out.impl()->tensor = std::get<0>(r);
    saved.lse.impl()->tensor = std::get<1>(r);
    saved.cum_q.impl()->tensor = std::get<2>(r);
    saved.cum_k.impl()->tensor = std::get<3>(r);
    bw_meta->max_q = std::get<4>(r).expect_int();
    bw_meta->max_k = std::get<5>(r).expect_int();
    saved.seed.impl()->tensor = std::get<6>(r);
    saved.offset.impl()->tensor = std::get<7>(r);
    return std::get<0>(r).transpose(1, 2);
  }
  CS_ASSERT_TRUE(args.dropout_p == 0.0, "attention dropout needs the CUDA half/bf16 path");
  auto r = sdpa_math_forward(q, k, v, args.is_causal, scale);
  saved.out.impl()->tensor = r.out;
  saved.lse.impl()->tensor = r.lse;
  return r.out.transpose(1, 2);
}

std::array<at::Tensor, 3> attention_backward_body(const at::Tensor &dout4, const at::Tensor &q4, const at::Tensor &k4,
                                                  const at::Tensor &v4,
                                                  const ScaledDotProductAttention::State::Args &args,
                                                  const ScaledDotProductAttention::State::Backward &bw) {
  const at::Tensor q = q4.transpose(1, 2), k = k4.transpose(1, 2), v = v4.transpose(1, 2);
  const at::Tensor dout = dout4.transpose(1, 2);
  const double scale = resolve_scale(args.scale, q.size(-1));
  const at::Tensor &out = bw.out.impl()->tensor;
  const at::Tensor &lse = bw.logsumexp.impl()->tensor;
  const bool own_forward = bw.out.impl()->companion.defined();
  if (library_flash_ok(q) && use_cudnn_engine() && q.size(-1) <= 128 && !own_forward) {
    auto r = at::_scaled_dot_product_cudnn_attention_backward(
        dout.to(q.scalar_type()), q, k, v, out, lse, bw.philox_seed.impl()->tensor, bw.philox_offset.impl()->tensor,
        at::Tensor{}, bw.cum_seq_q.impl()->tensor, bw.cum_seq_k.impl()->tensor, bw.max_q, bw.max_k, args.dropout_p,
        args.is_causal, scale);
    return {std::get<0>(r).transpose(1, 2), std::get<1>(r).transpose(1, 2), std::get<2>(r).transpose(1, 2)};
  }
  if (library_flash_ok(q)) {
    auto r = at::_scaled_dot_product_flash_attention_backward(
        dout.to(q.scalar_type()), q, k, v, out, lse, bw.cum_seq_q.impl()->tensor, bw.cum_seq_k.impl()->tensor,
        bw.max_q, bw.max_k, args.dropout_p, args.is_causal, bw.philox_seed.impl()->tensor,
        bw.philox_offset.impl()->tensor, scale);
    return {std::get<0>(r).transpose(1, 2), std::get<1>(r).transpose(1, 2), std::get<2>(r).transpose(1, 2)};
  }
  auto r = sdpa_math_backward(dout, q, k, v, out, lse, args.is_causal, scale);
  return {r[0].transpose(1, 2), r[1].transpose(1, 2), r[2].transpose(1, 2)};
}

void attention_release(ScaledDotProductAttention::State::Backward &b) {
  b.query.reset();
  b.key.reset();
  b.value.reset();
  b.qkv.reset();
  b.out.reset();
  b.logsumexp.reset();
  b.cum_seq_q.reset();
  b.cum_seq_k.reset();
  b.philox_seed.reset();
  b.philox_offset.reset();
}
}  // namespace

Tensor ScaledDotProductAttention::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                          const ReadOnlyTensor &query, const ReadOnlyTensor &key,
                                          const ReadOnlyTensor &value) {
  Tensor output;
  Saved saved;
  auto &b = state->backward;
  b.query = query;
  b.key = key;
  b.value = value;
  b.packed = false;
  b.out = saved.out;
  b.logsumexp = saved.lse;
  b.cum_seq_q = saved.cum_q;
  b.cum_seq_k = saved.cum_k;
  b.philox_seed = saved.seed;
  b.philox_offset = saved.offset;
  submit(scheduler, "cs::compute::ScaledDotProductAttention::forward", Task::Impl::kMain, Task::Impl::kCompute,
         {output, saved.out, saved.lse, saved.cum_q, saved.cum_k, saved.seed, saved.offset}, {query, key, value},
         [query, key, value, state, saved, output](const FnTask &) {
           output.impl()->tensor = attention_forward_body(query.impl()->tensor, key.impl()->tensor,
                                                          value.impl()->tensor, state->args, &state->backward, saved);
         });
  return output;
}

std::array<Tensor, 3> ScaledDotProductAttention::backward(const Scheduler &scheduler,
                                                          const std::shared_ptr<State> &state,
                                                          const ReadOnlyTensor &grad_out) {
  Tensor dq, dk, dv;
  auto &b = state->backward;
  submit(scheduler, "cs::compute::ScaledDotProductAttention::backward", Task::Impl::kMain, Task::Impl::kCompute,
         {dq, dk, dv},
         {grad_out, b.query, b.key, b.value, b.out, b.logsumexp, b.cum_seq_q, b.cum_seq_k, b.philox_seed,
          b.philox_offset},
         [grad_out, bw = state->backward, args = state->args, dq, dk, dv](const FnTask &) {
           auto r = attention_backward_body(grad_out.impl()->tensor, bw.query.impl()->tensor, bw.key.impl()->tensor,
                                            bw.value.impl()->tensor, args, bw);
           dq.impl()->tensor = r[0];
           dk.impl()->tensor = r[1];
           dv.impl()->tensor = r[2];
         });
  attention_release(b);
  return {dq, dk, dv};
}

Tensor ScaledDotProductAttention::forward_packed(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                                 const ReadOnlyTensor &qkv, int64_t num_heads) {
  Tensor output;
  Saved saved;
  auto &b = state->backward;
  b.qkv = qkv;
  b.packed = true;
  b.max_q = num_heads;  // reused as scratch until the task overwrites it; heads are re-derived from shapes
  b.out = saved.out;
  b.logsumexp = saved.lse;
  b.cum_seq_q = saved.cum_q;
  b.cum_seq_k = saved.cum_k;
  b.philox_seed = saved.seed;
  b.philox_offset = saved.offset;
  submit(scheduler, "cs::compute::ScaledDotProductAttention::forward_packed", Task::Impl::kMain, Task::Impl::kCompute,
         {output, saved.out, saved.lse, saved.cum_q, saved.cum_k, saved.seed, saved.offset}, {qkv},
         [qkv, state, saved, output, num_heads](const FnTask &) {
           const at::Tensor &x = qkv.impl()->tensor;  // [B,T,3*H*D]
           CS_ASSERT_TRUE(x.dim() == 3 && x.size(2) % (3 * num_heads) == 0, "packed qkv must be [B,T,3*H*D]");
           const int64_t B = x.size(0), T = x.size(1), D = x.size(2) / (3 * num_heads);
           if (use_own_forward() && x.is_cuda() && x.scalar_type() == at::kBFloat16 && fused_enabled() && x.is_contiguous() &&
               state->args.dropout_p == 0.0) {
             at::Tensor o = at::empty({B, T, num_heads * D}, x.options());
             at::Tensor lse = at::empty({B, num_heads, T}, x.options().dtype(at::kFloat));
             const int code = kernels::attention_forward_packed(current_stream(), x.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), B,
                                                                T, num_heads, D,
                                                                static_cast<float>(resolve_scale(state->args.scale, D)),
                                                                state->args.is_causal ? 1 : 0);
             if (code == 0) {
               saved.out.impl()->tensor = o.view({B, T, num_heads, D}).transpose(1, 2);  // [B,H,T,D] view
               saved.lse.impl()->tensor = lse;
               saved.cum_q.impl()->tensor = at::Tensor{};
               saved.cum_k.impl()->tensor = at::Tensor{};
               state->backward.max_q = T;
               state->backward.max_k = T;
               saved.seed.impl()->tensor = at::zeros({}, x.options().dtype(at::kLong));
               saved.offset.impl()->tensor = at::zeros({}, x.options().dtype(at::kLong));
               saved.out.impl()->companion = at::empty({0}, x.options());  // marks "own forward"
               output.impl()->tensor = o;
               return;
             }
             CS_ASSERT_TRUE(code == -1, "attention_forward_packed failed: ", cuda_error_string(code));
           }
           if (x.is_cuda() && x.scalar_type() == at::kBFloat16 && fused_enabled())
             note_library_fallback("ScaledDotProductAttention::forward_packed",
                                   use_own_forward() ? str_cat("T=", T, " D=", D, " causal=", state->args.is_causal, " dropout=",
                                                               state->args.dropout_p).c_str()
                                                     : "library engine selected by CS_ATTENTION_ENGINE");
           const at::Tensor x5 = x.view({B, T, 3, num_heads, D});
           at::Tensor o = attention_forward_body(x5.select(2, 0), x5.select(2, 1), x5.select(2, 2), state->args,
                                                 &state->backward, saved);
           output.impl()->tensor = o.contiguous().view({B, T, num_heads * D});
         });
  return output;
}

Tensor ScaledDotProductAttention::backward_packed(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                                  const ReadOnlyTensor &grad_out) {
  Tensor dqkv;
  auto &b = state->backward;
  CS_ASSERT_TRUE(b.packed, "backward_packed needs a forward_packed call first");
  submit(scheduler, "cs::compute::ScaledDotProductAttention::backward_packed", Task::Impl::kMain, Task::Impl::kCompute,
         {dqkv}, {grad_out, b.qkv, b.out, b.logsumexp, b.cum_seq_q, b.cum_seq_k, b.philox_seed, b.philox_offset},
         [grad_out, bw = state->backward, args = state->args, dqkv](const FnTask &) {
           const at::Tensor &x = bw.qkv.impl()->tensor;
           const at::Tensor &o = bw.out.impl()->tensor;  // [B,H,T,D]
           const int64_t B = x.size(0), T = x.size(1), H = o.size(1), D = o.size(3);
           const at::Tensor &go = grad_out.impl()->tensor;
           if (bw.out.impl()->companion.defined() && x.is_cuda() && x.is_contiguous() && go.is_contiguous() &&
               go.scalar_type() == at::kBFloat16 && fused_enabled()) {
             // the forward ran on this library's kernel: its output buffer is [B,T,H,D] and the backward kernels
             // read the packed qkv and write the packed gradient directly
             const at::Tensor o_bthd = o.transpose(1, 2);
             if (o_bthd.is_contiguous()) {
               at::Tensor packed = at::empty({B, T, 3 * H * D}, x.options());
               at::Tensor delta = at::empty({3, B, H, T}, x.options().dtype(at::kFloat));
               const int code = kernels::attention_backward_packed(
                   current_stream(), x.data_ptr(), o_bthd.data_ptr(), go.data_ptr(), bw.logsumexp.impl()->tensor.data_ptr<float>(),
                   delta.data_ptr<float>(), packed.data_ptr(), B, T, H, D, static_cast<float>(resolve_scale(args.scale, D)),
                   args.is_causal ? 1 : 0);
               if (code == 0) {
                 dqkv.impl()->tensor = packed;
                 return;
               }
               CS_ASSERT_TRUE(code == -1, "attention_backward_packed failed: ", cuda_error_string(code));
             }
           }
           const at::Tensor x5 = x.view({B, T, 3, H, D});
           const at::Tensor do4 = go.reshape({B, T, H, D});
           auto r = attention_backward_body(do4, x5.select(2, 0), x5.select(2, 1), x5.select(2, 2), args, bw);
           at::Tensor packed = at::empty({B, T, 3, H, D}, x.options());
           // r[i] are [B,T,H,D] tensors, either contiguous or views of [B,H,T,D] buffers (depends on
           // the library engine); one kernel interleaves all three
           const bool bthd = r[0].is_contiguous() && r[1].is_contiguous() && r[2].is_contiguous();
           const at::Tensor dq = r[0].transpose(1, 2), dk = r[1].transpose(1, 2), dv = r[2].transpose(1, 2);
           const bool bhtd = dq.is_contiguous() && dk.is_contiguous() && dv.is_contiguous();
           if (x.is_cuda() && x.scalar_type() == at::kBFloat16 && fused_enabled() && D % 8 == 0 && (bthd || bhtd)) {
             check_kernel(kernels::pack_qkv(current_stream(), r[0].data_ptr(), r[1].data_ptr(), r[2].data_ptr(),
                                            packed.data_ptr(), B, H, T, D, bthd ? 1 : 0),
                          "pack_qkv");
           } else {
             packed.select(2, 0).copy_(r[0]);
             packed.select(2, 1).copy_(r[1]);
             packed.select(2, 2).copy_(r[2]);
           }
           dqkv.impl()->tensor = packed.view({B, T, 3 * H * D});
         });
  attention_release(b);
  return dqkv;
}

// ======================================================================================
// Utils
// ======================================================================================
namespace {
TensorOptions on_device(const Scheduler &scheduler, TensorOptions options) {
  return options.has_device() ? options : options.device(scheduler.device());
}

template <typename F>
Tensor produce(const Scheduler &scheduler, const char *name, std::vector<ReadOnlyTensor> inputs, F &&fn) {
  Tensor out;
  submit(scheduler, name, Task::Impl::kMain, Task::Impl::kCompute, {out}, std::move(inputs),
         [out, fn = std::forward<F>(fn)](const FnTask &) { out.impl()->tensor = fn(); });
  return out;
}

template <typename F>
void mutate(const Scheduler &scheduler, const char *name, const Tensor &target, F &&fn) {
  submit(scheduler, name, Task::Impl::kMain, Task::Impl::kCompute, {target}, {},
         [target, fn = std::forward<F>(fn)](const FnTask &) {
           fn(target.impl()->tensor);
           ++target.impl()->version;
         });
}
}  // namespace

Tensor Utils::sum(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef dim, bool keep_dim,
                  optional<at::ScalarType> dtype) {
  return produce(scheduler, "cs::compute::Utils::sum", {input},
                 [input, d = IntArray(dim.begin(), dim.end()), keep_dim, dtype] {
                   return at::sum(input.impl()->tensor, d, keep_dim, dtype);
                 });
}
Tensor Utils::sum(const Scheduler &scheduler, const ReadOnlyTensor &input, int64_t dim, bool keep_dim,
                  optional<at::ScalarType> dtype) {
  return sum(scheduler, input, IntArrayRef{dim}, keep_dim, dtype);
}
Tensor Utils::range(const Scheduler &scheduler, const Scalar &start, const Scalar &end, TensorOptions options) {
  options = on_device(scheduler, options);
  return produce(scheduler, "cs::compute::Utils::range", {}, [=] { return at::range(start, end, options); });
}
Tensor Utils::arange(const Scheduler &scheduler, const Scalar &start, const Scalar &end, TensorOptions options) {
  options = on_device(scheduler, options);
  return produce(scheduler, "cs::compute::Utils::arange", {}, [=] { return at::arange(start, end, options); });
}
Tensor Utils::arange(const Scheduler &scheduler, const Scalar &start, const Scalar &end, const Scalar &step,
                     TensorOptions options) {
  options = on_device(scheduler, options);
  return produce(scheduler, "cs::compute::Utils::arange", {}, [=] { return at::arange(start, end, step, options); });
}
Tensor Utils::randint(const Scheduler &scheduler, int64_t low, int64_t high, IntArrayRef size, TensorOptions options) {
  options = on_device(scheduler, options);
  return produce(scheduler, "cs::compute::Utils::randint", {},
                 [=, s = IntArray(size.begin(), size.end())] { return at::randint(low, high, s, options); });
}
#define CS_FACTORY(fname)                                                                              \
  Tensor Utils::fname(const Scheduler &scheduler, IntArrayRef size, TensorOptions options) {           \
    options = on_device(scheduler, options);                                                           \
    return produce(scheduler, "cs::compute::Utils::" #fname, {},                                       \
                   [=, s = IntArray(size.begin(), size.end())] { return at::fname(s, options); });     \
  }                                                                                                    \
  Tensor Utils::fname##_like(const Scheduler &scheduler, const ReadOnlyTensor &src) {                  \
    return produce(scheduler, "cs::compute::Utils::" #fname "_like", {src},                            \
                   [src] { return at::fname##_like(src.impl()->tensor); });                            \
  }
CS_FACTORY(empty)
CS_FACTORY(ones)
CS_FACTORY(zeros)
CS_FACTORY(rand)
CS_FACTORY(randn)
#undef CS_FACTORY

std::vector<Tensor> Utils::split(const Scheduler &scheduler, const ReadOnlyTensor &src, int64_t split_size,
                                 int64_t dim) {
  CS_ASSERT_TRUE(src.defined(), "Utils::split needs a materialised source to know its extent");
  const int64_t extent = src.size(dim < 0 ? dim + static_cast<int64_t>(src.sizes().size()) : dim);
  const int64_t pieces = (extent + split_size - 1) / split_size;
  std::vector<Tensor> outs(static_cast<size_t>(pieces));
  submit(scheduler, "cs::compute::Utils::split", Task::Impl::kMain, Task::Impl::kCompute, outs, {src},
         [outs, src, split_size, dim](const FnTask &) {
           auto parts = at::split(src.impl()->tensor, split_size, dim);
           CS_ASSERT_TRUE(parts.size() == outs.size(), "split produced an unexpected number of pieces");
           for (size_t i = 0; i < parts.size(); ++i) outs[i].impl()->tensor = parts[i];
         });
  return outs;
}
Tensor Utils::view(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef size) {
  return produce(scheduler, "cs::compute::Utils::view", {input}, [input, s = IntArray(size.begin(), size.end())] {
    const at::Tensor &t = input.impl()->tensor;
    return t.is_contiguous() ? t.view(s) : t.reshape(s);
  });
}
Tensor Utils::as_strided(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef size, IntArrayRef stride,
                         optional<int64_t> storage_offset) {
  return produce(scheduler, "cs::compute::Utils::as_strided", {input},
                 [input, s = IntArray(size.begin(), size.end()), st = IntArray(stride.begin(), stride.end()),
                  storage_offset] { return at::as_strided(input.impl()->tensor, s, st, storage_offset); });
}
Tensor Utils::broadcast_to(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef size) {
  return produce(scheduler, "cs::compute::Utils::broadcast_to", {input},
                 [input, s = IntArray(size.begin(), size.end())] { return at::broadcast_to(input.impl()->tensor, s); });
}
Tensor Utils::cat(const Scheduler &scheduler, const std::vector<ReadOnlyTensor> &input, int64_t dim) {
  return produce(scheduler, "cs::compute::Utils::cat", input, [input, dim] {
    std::vector<at::Tensor> parts;
    parts.reserve(input.size());
    for (auto &t : input) parts.push_back(t.impl()->tensor);
    return at::cat(parts, dim);
  });
}
Tensor Utils::add(const Scheduler &scheduler, const ReadOnlyTensor &x, const ReadOnlyTensor &y) {
  return produce(scheduler, "cs::compute::Utils::add", {x, y}, [x, y] {
    const at::Tensor &a = x.impl()->tensor;
    const at::Tensor &b = y.impl()->tensor;
    if (a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && fused_enabled() &&
        a.is_contiguous() && b.is_contiguous() && a.sizes() == b.sizes() && a.numel() % 8 == 0) {
      at::Tensor out = at::empty_like(a);
      check_kernel(kernels::add_bf16(current_stream(), a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel()), "add_bf16");
      return out;
    }
    return at::add(a, b);
  });
}
void Utils::zero_(const Scheduler &scheduler, const Tensor &tensor) {
  mutate(scheduler, "cs::compute::Utils::zero_", tensor, [](at::Tensor &t) { t.zero_(); });
}
void Utils::uniform_(const Scheduler &scheduler, const Tensor &tensor, double from, double to) {
  mutate(scheduler, "cs::compute::Utils::uniform_", tensor, [from, to](at::Tensor &t) { t.uniform_(from, to); });
}
void Utils::normal_(const Scheduler &scheduler, const Tensor &tensor, double mean, double std) {
  mutate(scheduler, "cs::compute::Utils::normal_", tensor, [mean, std](at::Tensor &t) { t.normal_(mean, std); });
}
Tensor Utils::clone(const Scheduler &scheduler, const Tensor &tensor) {
  return produce(scheduler, "cs::compute::Utils::clone", {tensor}, [tensor] { return tensor.impl()->tensor.clone(); });
}
Tensor Utils::to(const Scheduler &scheduler, const ReadOnlyTensor &input, TensorOptions options) {
  return produce(scheduler, "cs::compute::Utils::to", {input}, [input, options] { return input.impl()->tensor.to(options); });
}
Tensor Utils::linalg_vector_norm(const Scheduler &scheduler, const ReadOnlyTensor &self, const Scalar &ord,
                                 at::OptionalIntArrayRef dim, bool keepdim, optional<at::ScalarType> dtype) {
  optional<IntArray> d;
  if (dim.has_value()) d = IntArray(dim->begin(), dim->end());
  return produce(scheduler, "cs::compute::Utils::linalg_vector_norm", {self}, [self, ord, d, keepdim, dtype] {
    return at::linalg_vector_norm(self.impl()->tensor, ord,
                                  d.has_value() ? at::OptionalIntArrayRef{IntArrayRef{*d}} : c10::nullopt, keepdim, dtype);
  });
}

Tensor Utils::clip_grad_norm_(const Scheduler &scheduler, const std::vector<Tensor> &tensors, double max_norm,
                              double norm_type) {
  Tensor total;
  std::vector<Tensor> outs{total};
  std::vector<ReadOnlyTensor> ins;
  for (auto &t : tensors) {
    outs.push_back(t);
    ins.push_back(t);
  }
  submit(scheduler, "cs::compute::Utils::clip_grad_norm_", Task::Impl::kMain, Task::Impl::kCompute, outs, ins,
         [tensors, total, max_norm, norm_type](const FnTask &task) {
           std::vector<at::Tensor> grads;
           for (auto &t : tensors)
             if (t.impl()->tensor.defined()) grads.push_back(t.impl()->tensor);
           CS_ASSERT_TRUE(!grads.empty(), "clip_grad_norm_ needs at least one defined gradient");
           bool fused = norm_type == 2.0 && fused_enabled();
           for (auto &g : grads)
             fused = fused && g.is_cuda() && g.is_contiguous() && dtype_code(g.scalar_type()) >= 0 &&
                     dtype_code(g.scalar_type()) <= 1;
           if (fused) {
             at::Tensor work = at::zeros({3}, grads[0].options().dtype(at::kFloat));  // sumsq, coef, norm
             task.intermediate().push_back(work);
             float *w = work.data_ptr<float>();
             for (auto &g : grads)
               check_kernel(kernels::sum_squares(current_stream(), g.data_ptr(), dtype_code(g.scalar_type()), g.numel(), w),
                            "sum_squares");
             check_kernel(kernels::clip_coefficient(current_stream(), w, static_cast<float>(max_norm), w + 1, w + 2),
                          "clip_coefficient");
             for (auto &g : grads)
               check_kernel(kernels::scale_by_device_scalar(current_stream(), g.data_ptr(), dtype_code(g.scalar_type()),
                                                            g.numel(), w + 1),
                            "scale_by_device_scalar");
             total.impl()->tensor = work.narrow(0, 2, 1).reshape({});
             return;
           }
           std::vector<at::Tensor> norms;
           for (auto &g : grads) norms.push_back(at::linalg_vector_norm(g, norm_type).to(at::kFloat).reshape({1}));
           at::Tensor n = at::linalg_vector_norm(at::cat(norms), norm_type);
           at::Tensor coef = at::clamp_max(max_norm / (n + 1e-6), 1.0);
           for (auto &g : grads) g.mul_(coef.to(g.scalar_type()));
           total.impl()->tensor = n;
         });
  return total;
}

// ======================================================================================
// Init
// ======================================================================================
namespace {
double gain_of(Nonlinearity nl, double a) {
  switch (nl) {
    case Nonlinearity::kLinear:
    case Nonlinearity::kSigmoid: return 1.0;
    case Nonlinearity::kTanh: return 5.0 / 3.0;
    case Nonlinearity::kReLU: return std::sqrt(2.0);
    case Nonlinearity::kLeakyReLU: return std::sqrt(2.0 / (1.0 + a * a));
  }
  return 1.0;
}
double fan_of(const at::Tensor &t, FanMode mode) {
  CS_ASSERT_TRUE(t.dim() >= 2, "fan in/out needs at least 2 dimensions");
  int64_t receptive = 1;
  for (int64_t i = 2; i < t.dim(); ++i) receptive *= t.size(i);
  return static_cast<double>((mode == FanMode::kFanIn ? t.size(1) : t.size(0)) * receptive);
}
}  // namespace

void Init::kaiming_normal_(const Scheduler &scheduler, const Tensor &tensor, double a, FanMode mode,
                           Nonlinearity nonlinearity) {
  mutate(scheduler, "cs::compute::Init::kaiming_normal_", tensor, [a, mode, nonlinearity](at::Tensor &t) {
    t.normal_(0, gain_of(nonlinearity, a) / std::sqrt(fan_of(t, mode)));
  });
}
void Init::kaiming_uniform_(const Scheduler &scheduler, const Tensor &tensor, double a, FanMode mode,
                            Nonlinearity nonlinearity) {
  mutate(scheduler, "cs::compute::Init::kaiming_uniform_", tensor, [a, mode, nonlinearity](at::Tensor &t) {
    const double bound = std::sqrt(3.0) * gain_of(nonlinearity, a) / std::sqrt(fan_of(t, mode));
    t.uniform_(-bound, bound);
  });
}
}  // namespace cs::compute
