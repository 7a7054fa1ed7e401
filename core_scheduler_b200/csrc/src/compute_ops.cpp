// SPDX-License-Identifier: Apache-2.0
// Parameter-owning and activation ops (Linear, GeluLinear, LayerNorm, GeLU, Embedding,
// CrossEntropy, LinearCrossEntropy, ScaledDotProductAttention). See cs/compute.h.
//
// Reference behaviour studied in src/compute/{linear,gelu_linear_cudnn,layer_norm,gelu,
// embedding,cross_entropy,sdpa_flash_attn,sdpa_cudnn}.cpp of the reference project: forward
// saves what backward needs in the state, backward_input runs on the main stream,
// backward_parameter on the assist stream, gradients are assigned on the first micro-step
// and accumulated afterwards, saved activations are released once consumed.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <cmath>
#include <mutex>
#include <set>

#include "cs/compute.h"
#include "kernels/api.h"
#include "op_common.h"

namespace cs::compute {
namespace {
std::atomic<int> g_backend{static_cast<int>(Backend::kFused)};
}
void set_backend(Backend backend) { g_backend.store(static_cast<int>(backend)); }
Backend get_backend() { return static_cast<Backend>(g_backend.load()); }

namespace detail {
bool fused_enabled() { return get_backend() == Backend::kFused; }

void *current_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void check_kernel(int code, const char *what) {
  CS_ASSERT_TRUE(code == 0, "kernel launch `", what, "` failed: ", cuda_error_string(code));
}

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return 0;
    case at::kBFloat16: return 1;
    case at::kHalf: return 2;
    default: return -1;
  }
}

void store_grad(const Tensor &slot, const at::Tensor &value, at::ScalarType store_dtype) {
  auto &impl = *slot.impl();
  if (!impl.tensor.defined()) {
    impl.tensor = value.scalar_type() == store_dtype ? value : value.to(store_dtype);
    impl.fresh = false;
    return;
  }
  if (impl.fresh) {
    impl.tensor.copy_(value.view_as(impl.tensor));
    impl.fresh = false;
    return;
  }
  impl.tensor.add_(value.view_as(impl.tensor));
}

bool grad_slot_ready_for_fused(const Tensor &slot) {
  const auto &impl = *slot.impl();
  return impl.tensor.defined() && impl.tensor.scalar_type() == at::kFloat && impl.tensor.is_contiguous();
}

at::Tensor as2d(const at::Tensor &t) { return t.reshape({-1, t.size(-1)}).contiguous(); }

namespace {
std::atomic<int64_t> g_library_fallbacks{0};
}
int64_t library_fallback_count() { return g_library_fallbacks.load(); }
void note_library_fallback(const char *op, const char *reason) {
  g_library_fallbacks.fetch_add(1);
  static std::mutex mu;
  static std::set<std::string> seen;
  const std::string key = str_cat(op, ": ", reason);
  std::lock_guard<std::mutex> lock{mu};
  if (!seen.insert(key).second) return;
  logger().warn("library fallback in ", key, " (this library's sm_100a kernel does not cover the case; reported once)");
}

// D = A[M,K] * B[N,K]^T through the tcgen05 kernel; false when the shape is not covered.
bool fused_gemm(const kernels::GemmArgs &args) {
  const int code = kernels::gemm_bf16(current_stream(), args);
  if (code == -1) {
    note_library_fallback("gemm_bf16", str_cat("m=", args.m, " n=", args.n, " k=", args.k, " layout=", args.layout).c_str());
    return false;
  }
  check_kernel(code, "gemm_bf16");
  return true;
}
}  // namespace detail
using namespace detail;
int64_t library_fallbacks() { return detail::library_fallback_count(); }

void bump_version(const Tensor &parameter) { ++parameter.impl()->version; }

namespace {
// The tensor a bf16 kernel should read for a parameter: its bf16 working copy when one exists
// and is current (it is the only complete copy under a sharded optimizer, where the fp32 master
// is authoritative only inside the owner's shard), else the parameter itself.
const at::Tensor &kernel_view(const ReadOnlyTensor &parameter) {
  const auto &impl = *parameter.impl();
  if (impl.lp.defined() && impl.lp_version == impl.version && impl.lp.scalar_type() == at::kBFloat16) return impl.lp;
  return impl.tensor;
}
}  // namespace

at::Tensor working_copy(const ReadOnlyTensor &parameter, at::ScalarType dtype) {
  auto &impl = *parameter.impl();
  if (impl.tensor.scalar_type() == dtype) return impl.tensor;
  if (impl.lp.defined() && impl.lp.scalar_type() == dtype) {
    if (impl.lp_version != impl.version) {
      impl.lp.copy_(impl.tensor);
      impl.lp_version = impl.version;
    }
    return impl.lp;
  }
  impl.lp = impl.tensor.to(dtype);
  impl.lp_version = impl.version;
  return impl.lp;
}

at::Tensor working_copy_transposed(const ReadOnlyTensor &parameter, at::ScalarType dtype) {
  auto &impl = *parameter.impl();
  CS_ASSERT_TRUE(impl.tensor.dim() == 2, "transposed working copies exist for matrices only");
  if (impl.lp_t.defined() && impl.lp_t.scalar_type() == dtype && impl.lp_t_version == impl.version) return impl.lp_t;
  const auto rows = impl.tensor.size(0), cols = impl.tensor.size(1);
  if (!impl.lp_t.defined() || impl.lp_t.scalar_type() != dtype)
    impl.lp_t = at::empty({cols, rows}, impl.tensor.options().dtype(dtype));
  const int src_code = dtype_code(impl.tensor.scalar_type());
  if (impl.tensor.is_cuda() && dtype == at::kBFloat16 && src_code >= 0 && impl.tensor.is_contiguous()) {
    check_kernel(kernels::transpose_cast_to_bf16(current_stream(), impl.tensor.data_ptr(), src_code,
                                                 impl.lp_t.data_ptr(), rows, cols),
                 "transpose_cast_to_bf16");
  } else {
    impl.lp_t.copy_(impl.tensor.t());
  }
  impl.lp_t_version = impl.version;
  return impl.lp_t;
}

// ======================================================================================
// Linear
// ======================================================================================
namespace {
template <typename S>
OrderedDict<std::string, Tensor> wb_parameters(const S &s) {
  OrderedDict<std::string, Tensor> d;
  d.insert("weight", s.forward.weight);
  if (s.args.bias) d.insert("bias", s.forward.bias);
  return d;
}
template <typename S>
OrderedDict<std::string, Tensor> wb_gradients(const S &s) {
  OrderedDict<std::string, Tensor> d;
  d.insert("weight", s.forward.grad_weight);
  if (s.args.bias) d.insert("bias", s.forward.grad_bias);
  return d;
}
template <typename S>
OrderedDict<std::string, module::State::Increment> wb_increments(const S &s) {
  OrderedDict<std::string, module::State::Increment> d;
  d.insert("weight", {s.forward.weight, s.forward.grad_weight});
  if (s.args.bias) d.insert("bias", {s.forward.bias, s.forward.grad_bias});
  return d;
}

struct LinearInit {
  Tensor weight, bias;
};
LinearInit init_linear_parameters(const Scheduler &scheduler, const Linear::Options &options, const char *name) {
  LinearInit out;
  TensorOptions topt{};
  topt = topt.device(options.device().value_or(scheduler.device())).dtype(options.dtype().value_or(at::kFloat));
  std::vector<Tensor> outputs{out.weight};
  if (options.bias()) outputs.push_back(out.bias);
  const int64_t in = options.in_futures(), outf = options.out_futures();
  const bool with_bias = options.bias();
  submit(scheduler, name, Task::Impl::kMain, Task::Impl::kCompute, outputs, {},
         [w = out.weight, b = out.bias, topt, in, outf, with_bias](const FnTask &) {
           // kaiming-uniform with a = sqrt(5): U(-1/sqrt(fan_in), 1/sqrt(fan_in)) for the weight as well
           const double bound = 1.0 / std::sqrt(static_cast<double>(in));
           w.impl()->tensor = at::empty({outf, in}, topt).uniform_(-bound, bound);
           ++w.impl()->version;
           if (with_bias) {
             b.impl()->tensor = at::empty({outf}, topt).uniform_(-bound, bound);
             ++b.impl()->version;
           }
         });
  return out;
}

// Chooses the compute dtype of a matmul-class op and stamps the autocast decision on the
// tensors so that backward (which may run outside the guard) repeats it.
at::ScalarType matmul_dtype(const Scheduler &scheduler, const ReadOnlyTensor &x, const Tensor &w, const Tensor &b) {
  const auto &impl = *scheduler.impl();
  if (impl.autocast_enabled) {
    for (const ReadOnlyTensor *t : {&x, static_cast<const ReadOnlyTensor *>(&w), static_cast<const ReadOnlyTensor *>(&b)}) {
      t->impl()->autocast_enabled = true;
      t->impl()->autocast_dtype = impl.autocast_dtype;
    }
    return impl.autocast_dtype;
  }
  w.impl()->autocast_enabled = false;
  return at::ScalarType::Undefined;  // decided from the tensors inside the task
}

at::Tensor cast_if(const at::Tensor &t, at::ScalarType dt) { return t.scalar_type() == dt ? t : t.to(dt); }

// Body of Linear-like forward: y = x W^T (+b) (+residual) with optional GELU companion.
void linear_forward_body(const ReadOnlyTensor &input, const Tensor &weight, const Tensor &bias, bool with_bias,
                         const ReadOnlyTensor *residual, bool gelu_dual, at::ScalarType amp_dt, const Tensor &output) {
  const at::Tensor &x = input.impl()->tensor;
  const at::ScalarType dt = amp_dt == at::ScalarType::Undefined ? x.scalar_type() : amp_dt;
  const at::Tensor xc = cast_if(x, dt);
  const at::Tensor wc = working_copy(weight, dt);
  at::Tensor bc;
  if (with_bias) bc = working_copy(bias, dt);
  if (xc.is_cuda() && dt == at::kBFloat16 && fused_enabled()) {
    const at::Tensor x2 = as2d(xc);
    auto out_sizes = xc.sizes().vec();
    out_sizes.back() = wc.size(0);
    at::Tensor y = at::empty(out_sizes, xc.options());
    at::Tensor y2, res2;
    kernels::GemmArgs g{};
    g.a = x2.data_ptr();
    g.b = wc.data_ptr();
    g.d = y.data_ptr();
    g.m = x2.size(0);
    g.n = wc.size(0);
    g.k = x2.size(1);
    g.lda = g.k;
    g.ldb = g.k;
    g.ldd = g.n;
    g.layout = kernels::kTN;
    g.bias = with_bias ? bc.data_ptr() : nullptr;
    g.epilogue = kernels::kEpiStoreBf16;
    if (residual) {
      res2 = cast_if(residual->impl()->tensor, dt).contiguous();
      g.aux = res2.data_ptr();
      g.epilogue = kernels::kEpiResidualBf16;
    } else if (gelu_dual) {
      y2 = at::empty(out_sizes, xc.options());
      g.d2 = y2.data_ptr();
      g.epilogue = kernels::kEpiGeluDual;
    }
    if (fused_gemm(g)) {
      output.impl()->tensor = y;
      output.impl()->companion = y2;
      return;
    }
  }
  at::Tensor y = at::linear(xc, wc, with_bias ? std::optional<at::Tensor>{bc} : std::nullopt);
  if (residual) y = y.add_(cast_if(residual->impl()->tensor, dt));
  output.impl()->tensor = y;
  output.impl()->companion = gelu_dual ? at::gelu(y) : at::Tensor{};
}

// dX = dY W  (optionally multiplied by GELU'(pre)).
at::Tensor linear_dgrad(const at::Tensor &dy_in, const Tensor &weight, at::ScalarType dt, const at::Tensor *pre) {
  const at::Tensor dy = cast_if(dy_in, dt);
  if (dy.is_cuda() && dt == at::kBFloat16 && fused_enabled()) {
    const at::Tensor wc = working_copy(weight, dt);  // [out, in], read as the MN-major B operand
    const at::Tensor dy2 = as2d(dy);
    auto out_sizes = dy.sizes().vec();
    out_sizes.back() = wc.size(1);
    at::Tensor dx = at::empty(out_sizes, dy.options());
    at::Tensor pre2;
    kernels::GemmArgs g{};
    g.a = dy2.data_ptr();
    g.b = wc.data_ptr();
    g.d = dx.data_ptr();
    g.m = dy2.size(0);
    g.n = wc.size(1);
    g.k = dy2.size(1);
    g.lda = g.k;
    g.ldb = g.n;
    g.ldd = g.n;
    g.layout = kernels::kTM;
    g.epilogue = kernels::kEpiStoreBf16;
    if (pre) {
      pre2 = cast_if(*pre, dt).contiguous();
      g.aux = pre2.data_ptr();
      g.epilogue = kernels::kEpiDGelu;
    }
    if (fused_gemm(g)) return dx;
  }
  at::Tensor dx = at::matmul(dy, working_copy(weight, dt));
  if (pre) dx = at::gelu_backward(dx, cast_if(*pre, dt));
  return dx;
}

// dW (+)= dY^T X into the gradient slot.
void linear_wgrad(const at::Tensor &dy_in, const at::Tensor &x_in, at::ScalarType dt, const Tensor &weight,
                  const Tensor &grad_slot) {
  const at::Tensor dy2 = as2d(cast_if(dy_in, dt));
  const at::Tensor x2 = as2d(cast_if(x_in, dt));
  const at::ScalarType store = weight.impl()->tensor.scalar_type();
  if (dy2.is_cuda() && dt == at::kBFloat16 && fused_enabled() && store == at::kFloat) {
    auto &slot = *grad_slot.impl();
    const bool had = slot.tensor.defined();
    if (!had) slot.tensor = at::empty_like(weight.impl()->tensor);
    if (grad_slot_ready_for_fused(grad_slot)) {
      kernels::GemmArgs g{};
      g.a = dy2.data_ptr();
      g.b = x2.data_ptr();
      g.d = slot.tensor.data_ptr();
      g.m = dy2.size(1);
      g.n = x2.size(1);
      g.k = dy2.size(0);
      g.lda = g.m;
      g.ldb = g.n;
      g.ldd = g.n;
      g.layout = kernels::kNT;
      g.epilogue = (!had || slot.fresh) ? kernels::kEpiStoreF32 : kernels::kEpiAccumF32;
      if (fused_gemm(g)) {
        slot.fresh = false;
        return;
      }
    }
    if (!had) slot.tensor = at::Tensor{};
  }
  store_grad(grad_slot, at::matmul(dy2.t(), x2), store);
}

void bias_grad(const at::Tensor &dy, const Tensor &bias, const Tensor &grad_slot) {
  const at::ScalarType store = bias.impl()->tensor.scalar_type();
  const at::Tensor dy2 = dy.reshape({-1, dy.size(-1)});
  store_grad(grad_slot, at::sum(dy2, {0}, false, store == at::kDouble ? at::kDouble : at::kFloat).to(store), store);
}

at::ScalarType backward_dtype(const Tensor &weight, const at::Tensor &dy) {
  return weight.impl()->autocast_enabled ? weight.impl()->autocast_dtype
                                         : (dy.scalar_type() == weight.impl()->tensor.scalar_type()
                                                ? dy.scalar_type()
                                                : dy.scalar_type());
}
}  // namespace

OrderedDict<std::string, Tensor> Linear::State::parameters() const { return wb_parameters(*this); }
OrderedDict<std::string, Tensor> Linear::State::gradients() const { return wb_gradients(*this); }
OrderedDict<std::string, module::State::Increment> Linear::State::increments() const { return wb_increments(*this); }
void Linear::State::zero_grad() {
  module::clear_gradient(forward.grad_weight);
  if (args.bias) module::clear_gradient(forward.grad_bias);
}

std::shared_ptr<Linear::State> Linear::init(const Scheduler &scheduler, const Options &options) {
  auto p = init_linear_parameters(scheduler, options, "cs::compute::Linear::init");
  return std::make_shared<State>(State::Forward{p.weight, p.bias}, State::Backward{},
                                 State::Args{options.bias(), options.gelu_epilogue()});
}

namespace {
Tensor linear_forward_impl(const Scheduler &scheduler, const std::shared_ptr<Linear::State> &state,
                           const ReadOnlyTensor &input, const ReadOnlyTensor *residual) {
  Tensor output;
  state->backward.input = input;
  const at::ScalarType amp_dt = matmul_dtype(scheduler, input, state->forward.weight, state->forward.bias);
  std::vector<ReadOnlyTensor> inputs{input, state->forward.weight};
  if (state->args.bias) inputs.push_back(state->forward.bias);
  std::optional<ReadOnlyTensor> res;
  if (residual) {
    res = *residual;
    inputs.push_back(*residual);
  }
  submit(scheduler, "cs::compute::Linear::forward", Task::Impl::kMain, Task::Impl::kCompute, {output}, inputs,
         [input, w = state->forward.weight, b = state->forward.bias, with_bias = state->args.bias, res,
          gelu = state->args.gelu_epilogue, amp_dt, output](const FnTask &) {
           linear_forward_body(input, w, b, with_bias, res ? &*res : nullptr, gelu, amp_dt, output);
         });
  return output;
}
}  // namespace

Tensor Linear::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input) {
  return linear_forward_impl(scheduler, state, input, nullptr);
}
Tensor Linear::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input,
                       const ReadOnlyTensor &residual) {
  return linear_forward_impl(scheduler, state, input, &residual);
}

Tensor Linear::backward_input(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                              const ReadOnlyTensor &grad_output) {
  Tensor grad_input;
  submit(scheduler, "cs::compute::Linear::backward_input", Task::Impl::kMain, Task::Impl::kCompute, {grad_input},
         {grad_output, state->forward.weight}, [grad_output, w = state->forward.weight, grad_input](const FnTask &) {
           const at::Tensor &dy = grad_output.impl()->tensor;
           grad_input.impl()->tensor = linear_dgrad(dy, w, backward_dtype(w, dy), nullptr);
         });
  return grad_input;
}

void Linear::backward_parameter(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                const ReadOnlyTensor &grad_output) {
  CS_ASSERT_TRUE(state->backward.input.defined(), "Linear::backward_parameter called without a saved forward input");
  submit(scheduler, "cs::compute::Linear::backward_parameter", Task::Impl::kAssist, Task::Impl::kCompute,
         {state->forward.grad_weight}, {grad_output, state->backward.input, state->forward.weight},
         [grad_output, x = state->backward.input, w = state->forward.weight,
          gw = state->forward.grad_weight](const FnTask &) {
           const at::Tensor &dy = grad_output.impl()->tensor;
           linear_wgrad(dy, x.impl()->tensor, backward_dtype(w, dy), w, gw);
         });
  if (state->args.bias) {
    submit(scheduler, "cs::compute::Linear::backward_bias", Task::Impl::kAssist, Task::Impl::kCompute,
           {state->forward.grad_bias}, {grad_output, state->forward.bias},
           [grad_output, b = state->forward.bias, gb = state->forward.grad_bias](const FnTask &) {
             bias_grad(grad_output.impl()->tensor, b, gb);
           });
  }
  state->backward.input.reset();  // the tasks hold their own references
}

// ======================================================================================
// GeluLinear
// ======================================================================================
OrderedDict<std::string, Tensor> GeluLinear::State::parameters() const { return wb_parameters(*this); }
OrderedDict<std::string, Tensor> GeluLinear::State::gradients() const { return wb_gradients(*this); }
OrderedDict<std::string, module::State::Increment> GeluLinear::State::increments() const { return wb_increments(*this); }
void GeluLinear::State::zero_grad() {
  module::clear_gradient(forward.grad_weight);
  if (args.bias) module::clear_gradient(forward.grad_bias);
}

std::shared_ptr<GeluLinear::State> GeluLinear::init(const Scheduler &scheduler, const Options &options) {
  auto p = init_linear_parameters(scheduler, options, "cs::compute::GeluLinear::init");
  return std::make_shared<State>(State::Forward{p.weight, p.bias}, State::Backward{}, State::Args{options.bias()});
}

namespace {
Tensor gelu_linear_forward_impl(const Scheduler &scheduler, const std::shared_ptr<GeluLinear::State> &state,
                                const ReadOnlyTensor &input, const ReadOnlyTensor *residual) {
  Tensor output;
  Tensor activated;
  state->backward.input = input;
  state->backward.activated = activated;
  state->backward.input_count = 2;  // released after both backward halves ran
  const at::ScalarType amp_dt = matmul_dtype(scheduler, input, state->forward.weight, state->forward.bias);
  std::vector<ReadOnlyTensor> inputs{input, state->forward.weight};
  if (state->args.bias) inputs.push_back(state->forward.bias);
  std::optional<ReadOnlyTensor> res;
  if (residual) {
    res = *residual;
    inputs.push_back(*residual);
  }
  submit(scheduler, "cs::compute::GeluLinear::forward", Task::Impl::kMain, Task::Impl::kCompute, {output, activated},
         inputs,
         [input, w = state->forward.weight, b = state->forward.bias, with_bias = state->args.bias, res, amp_dt, output,
          activated](const FnTask &) {
           const at::Tensor &x = input.impl()->tensor;
           const at::ScalarType dt = amp_dt == at::ScalarType::Undefined ? x.scalar_type() : amp_dt;
           at::Tensor act = input.impl()->companion;
           if (!act.defined() || act.scalar_type() != dt) {
             const at::Tensor xc = cast_if(x, dt).contiguous();
             if (xc.is_cuda() && dt == at::kBFloat16 && fused_enabled()) {
               act = at::empty_like(xc);
               check_kernel(kernels::gelu_forward(current_stream(), xc.data_ptr(), act.data_ptr(), xc.numel()),
                            "gelu_forward");
             } else {
               act = at::gelu(xc);
             }
           }
           activated.impl()->tensor = act;
           linear_forward_body(activated, w, b, with_bias, res ? &*res : nullptr, false, amp_dt, output);
         });
  return output;
}
}  // namespace

Tensor GeluLinear::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                           const ReadOnlyTensor &input) {
  return gelu_linear_forward_impl(scheduler, state, input, nullptr);
}
Tensor GeluLinear::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input,
                           const ReadOnlyTensor &residual) {
  return gelu_linear_forward_impl(scheduler, state, input, &residual);
}

namespace {
void gelu_linear_release(const std::shared_ptr<GeluLinear::State> &state) {
  if (--state->backward.input_count <= 0) {
    state->backward.input.reset();
    state->backward.activated.reset();
  }
}
}  // namespace

Tensor GeluLinear::backward_input(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                  const ReadOnlyTensor &grad_output) {
  CS_ASSERT_TRUE(state->backward.input.defined(), "GeluLinear::backward_input called without a saved forward input");
  Tensor grad_input;
  submit(scheduler, "cs::compute::GeluLinear::backward_input", Task::Impl::kMain, Task::Impl::kCompute, {grad_input},
         {grad_output, state->forward.weight, state->backward.input},
         [grad_output, w = state->forward.weight, x = state->backward.input, grad_input](const FnTask &) {
           const at::Tensor &dy = grad_output.impl()->tensor;
           grad_input.impl()->tensor = linear_dgrad(dy, w, backward_dtype(w, dy), &x.impl()->tensor);
         });
  gelu_linear_release(state);
  return grad_input;
}

void GeluLinear::backward_parameter(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                    const ReadOnlyTensor &grad_output) {
  CS_ASSERT_TRUE(state->backward.activated.impl()->tensor.defined() || state->backward.input.defined(),
                 "GeluLinear::backward_parameter called without a saved forward input");
  submit(scheduler, "cs::compute::GeluLinear::backward_parameter", Task::Impl::kAssist, Task::Impl::kCompute,
         {state->forward.grad_weight}, {grad_output, state->backward.activated, state->forward.weight},
         [grad_output, act = state->backward.activated, w = state->forward.weight,
          gw = state->forward.grad_weight](const FnTask &) {
           const at::Tensor &dy = grad_output.impl()->tensor;
           linear_wgrad(dy, act.impl()->tensor, backward_dtype(w, dy), w, gw);
         });
  if (state->args.bias) {
    submit(scheduler, "cs::compute::GeluLinear::backward_bias", Task::Impl::kAssist, Task::Impl::kCompute,
           {state->forward.grad_bias}, {grad_output, state->forward.bias},
           [grad_output, b = state->forward.bias, gb = state->forward.grad_bias](const FnTask &) {
             bias_grad(grad_output.impl()->tensor, b, gb);
           });
  }
  gelu_linear_release(state);
}

// ======================================================================================
// LayerNorm
// ======================================================================================
OrderedDict<std::string, Tensor> LayerNorm::State::parameters() const {
  OrderedDict<std::string, Tensor> d;
  d.insert("weight", forward.weight);
  if (args.bias) d.insert("bias", forward.bias);
  return d;
}
OrderedDict<std::string, Tensor> LayerNorm::State::gradients() const {
  OrderedDict<std::string, Tensor> d;
  d.insert("weight", forward.grad_weight);
  if (args.bias) d.insert("bias", forward.grad_bias);
  return d;
}
OrderedDict<std::string, module::State::Increment> LayerNorm::State::increments() const {
  OrderedDict<std::string, Increment> d;
  d.insert("weight", {forward.weight, forward.grad_weight});
  if (args.bias) d.insert("bias", {forward.bias, forward.grad_bias});
  return d;
}
void LayerNorm::State::zero_grad() {
  module::clear_gradient(forward.grad_weight);
  if (args.bias) module::clear_gradient(forward.grad_bias);
}

std::shared_ptr<LayerNorm::State> LayerNorm::init(const Scheduler &scheduler, const Options &options) {
  CS_ASSERT_TRUE(options.elementwise_affine(), "LayerNorm without elementwise_affine is not supported");
  Tensor weight, bias;
  TensorOptions topt{};
  topt = topt.device(options.device().value_or(scheduler.device())).dtype(options.dtype().value_or(at::kFloat));
  std::vector<Tensor> outs{weight};
  if (options.bias()) outs.push_back(bias);
  submit(scheduler, "cs::compute::LayerNorm::init", Task::Impl::kMain, Task::Impl::kCompute, outs, {},
         [weight, bias, topt, shape = options.normalized_shape(), with_bias = options.bias()](const FnTask &) {
           weight.impl()->tensor = at::ones(shape, topt);
           ++weight.impl()->version;
           if (with_bias) {
             bias.impl()->tensor = at::zeros(shape, topt);
             ++bias.impl()->version;
           }
         });
  return std::make_shared<State>(
      State::Forward{weight, bias}, State::Backward{},
      State::Args{options.normalized_shape(), options.eps(), options.elementwise_affine(), options.bias()});
}

namespace {
bool ln_fused_ok(const at::Tensor &x, const at::Tensor &w, size_t norm_dims, int64_t max_d = 8192) {
  if (!(x.is_cuda() && x.scalar_type() == at::kBFloat16 && fused_enabled() && norm_dims == 1)) return false;
  const int64_t d = x.size(-1);
  return d % 8 == 0 && d <= max_d && dtype_code(w.scalar_type()) >= 0 && dtype_code(w.scalar_type()) <= 1;
}
}  // namespace

Tensor LayerNorm::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                          const ReadOnlyTensor &input) {
  Tensor output, mean, rstd;
  state->backward.input = input;
  state->backward.mean = mean;
  state->backward.rstd = rstd;
  const bool amp = scheduler.impl()->autocast_enabled;
  if (amp) {
    input.impl()->autocast_enabled = true;
    input.impl()->autocast_dtype = scheduler.impl()->autocast_dtype;
  }
  std::vector<ReadOnlyTensor> inputs{input, state->forward.weight};
  if (state->args.bias) inputs.push_back(state->forward.bias);
  submit(scheduler, "cs::compute::LayerNorm::forward", Task::Impl::kMain, Task::Impl::kCompute, {output, mean, rstd},
         inputs,
         [input, w = state->forward.weight, b = state->forward.bias, args = state->args, output, mean, rstd,
          amp](const FnTask &) {
           const at::Tensor x = input.impl()->tensor.contiguous();
           const at::Tensor &wt = w.impl()->tensor;
           if (ln_fused_ok(x, wt, args.normalized_shape.size()) &&
               (!args.bias || b.impl()->tensor.scalar_type() == wt.scalar_type())) {
             const at::Tensor &wk = kernel_view(w);
             const at::Tensor &bk = args.bias ? kernel_view(b) : wk;
             if (wk.scalar_type() == bk.scalar_type()) {
             const int64_t d = x.size(-1), rows = x.numel() / d;
             at::Tensor y = at::empty_like(x);
             auto stat_sizes = x.sizes().vec();
             stat_sizes.back() = 1;
             at::Tensor m = at::empty(stat_sizes, x.options().dtype(at::kFloat));
             at::Tensor r = at::empty(stat_sizes, x.options().dtype(at::kFloat));
             check_kernel(kernels::layernorm_forward(current_stream(), x.data_ptr(), wk.data_ptr(),
                                                     args.bias ? bk.data_ptr() : nullptr, dtype_code(wk.scalar_type()),
                                                     y.data_ptr(), m.data_ptr<float>(), r.data_ptr<float>(), rows, d,
                                                     static_cast<float>(args.eps)),
                          "layernorm_forward");
             output.impl()->tensor = y;
             mean.impl()->tensor = m;
             rstd.impl()->tensor = r;
             return;
             }
           }
           // Library path. Low-precision inputs are normalised in fp32 and cast back.
           const bool upcast = x.scalar_type() != wt.scalar_type() || (amp && x.scalar_type() != at::kDouble &&
                                                                       x.scalar_type() != at::kFloat);
           const at::ScalarType ct = upcast ? at::kFloat : x.scalar_type();
           auto [y, m, r] = at::native_layer_norm(
               cast_if(x, ct), args.normalized_shape, cast_if(wt, ct),
               args.bias ? std::optional<at::Tensor>{cast_if(b.impl()->tensor, ct)} : std::nullopt, args.eps);
           output.impl()->tensor = cast_if(y, x.scalar_type());
           mean.impl()->tensor = m;
           rstd.impl()->tensor = r;
         });
  return output;
}

namespace {
struct LnBackwardPlan {
  bool want_input;
  bool want_params;
};

// One task computing dx and/or dγ/dβ. `grad_residual` (optional) is added to dx.
Tensor layer_norm_backward_task(const Scheduler &scheduler, const std::shared_ptr<LayerNorm::State> &state,
                                const ReadOnlyTensor &grad_output, const ReadOnlyTensor *grad_residual,
                                LnBackwardPlan plan, Task::Impl::Priority priority, const char *name) {
  Tensor grad_input;
  std::vector<Tensor> outs;
  if (plan.want_input) outs.push_back(grad_input);
  if (plan.want_params) {
    outs.push_back(state->forward.grad_weight);
    if (state->args.bias) outs.push_back(state->forward.grad_bias);
  }
  std::vector<ReadOnlyTensor> ins{grad_output, state->backward.input, state->backward.mean, state->backward.rstd,
                                  state->forward.weight};
  std::optional<ReadOnlyTensor> res;
  if (grad_residual) {
    res = *grad_residual;
    ins.push_back(*grad_residual);
  }
  submit(scheduler, name, priority, Task::Impl::kCompute, outs, ins,
         [grad_output, x_h = state->backward.input, mean = state->backward.mean, rstd = state->backward.rstd,
          w = state->forward.weight, b = state->forward.bias, gw = state->forward.grad_weight,
          gb = state->forward.grad_bias, args = state->args, grad_input, res, plan](const FnTask &task) {
           const at::Tensor dy = grad_output.impl()->tensor.contiguous();
           const at::Tensor x = x_h.impl()->tensor.contiguous();
           const at::Tensor &wt = w.impl()->tensor;
           const at::ScalarType store = wt.scalar_type();
           if (plan.want_input && plan.want_params && ln_fused_ok(x, wt, args.normalized_shape.size(), 2048) &&
               dy.scalar_type() == at::kBFloat16 && store == at::kFloat && args.bias) {
             const int64_t d = x.size(-1), rows = x.numel() / d;
             auto &sw = *gw.impl();
             auto &sb = *gb.impl();
             const bool had = sw.tensor.defined() && sb.tensor.defined();
             const bool accumulate = had && !sw.fresh;
             if (!had) {
               sw.tensor = at::empty_like(wt);
               sb.tensor = at::empty_like(wt);
             }
             at::Tensor dx = at::empty_like(x);
             at::Tensor scratch =
                 at::empty({2 * kernels::layernorm_backward_scratch_rows() * d}, x.options().dtype(at::kFloat));
             task.intermediate().push_back(scratch);
             at::Tensor r2;
             if (res) r2 = cast_if(res->impl()->tensor, at::kBFloat16).contiguous();
             const at::Tensor &wk = kernel_view(w);
             check_kernel(kernels::layernorm_backward(
                              current_stream(), dy.data_ptr(), x.data_ptr(), wk.data_ptr(), dtype_code(wk.scalar_type()),
                              mean.impl()->tensor.data_ptr<float>(), rstd.impl()->tensor.data_ptr<float>(),
                              res ? r2.data_ptr() : nullptr, dx.data_ptr(), sw.tensor.data_ptr<float>(),
                              sb.tensor.data_ptr<float>(), accumulate ? 1 : 0, scratch.data_ptr<float>(), rows, d),
                          "layernorm_backward");
             sw.fresh = false;
             sb.fresh = false;
             grad_input.impl()->tensor = dx;
             return;
           }
           const bool upcast = x.scalar_type() != store || x_h.impl()->autocast_enabled;
           const at::ScalarType ct = upcast && x.scalar_type() != at::kDouble ? at::kFloat : x.scalar_type();
           auto [dx, dgamma, dbeta] = at::native_layer_norm_backward(
               cast_if(dy, ct), cast_if(x, ct), args.normalized_shape, mean.impl()->tensor, rstd.impl()->tensor,
               cast_if(wt, ct), args.bias ? std::optional<at::Tensor>{cast_if(b.impl()->tensor, ct)} : std::nullopt,
               {plan.want_input, plan.want_params, plan.want_params && args.bias});
           if (plan.want_params) {
             store_grad(gw, dgamma, store);
             if (args.bias) store_grad(gb, dbeta, store);
           }
           if (plan.want_input) {
             at::Tensor out = cast_if(dx, dy.scalar_type());
             if (res) out = out.add(cast_if(res->impl()->tensor, out.scalar_type()));
             grad_input.impl()->tensor = out;
           }
         });
  return grad_input;
}

void ln_release(const std::shared_ptr<LayerNorm::State> &state) {
  state->backward.input.reset();
  state->backward.mean.reset();
  state->backward.rstd.reset();
}

bool ln_single_pass(const Scheduler &scheduler, const std::shared_ptr<LayerNorm::State> &state,
                    const ReadOnlyTensor &grad_output) {
  const auto &x = state->backward.input.impl()->tensor;
  return scheduler.device().is_cuda() && x.defined() &&
         ln_fused_ok(x, state->forward.weight.impl()->tensor, state->args.normalized_shape.size(), 2048) &&
         grad_output.impl()->tensor.scalar_type() == at::kBFloat16 &&
         state->forward.weight.impl()->tensor.scalar_type() == at::kFloat && state->args.bias;
}
}  // namespace

Tensor LayerNorm::backward_input(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                 const ReadOnlyTensor &grad_output) {
  return layer_norm_backward_task(scheduler, state, grad_output, nullptr, {true, false}, Task::Impl::kMain,
                                  "cs::compute::LayerNorm::backward_input");
}

void LayerNorm::backward_parameter(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                   const ReadOnlyTensor &grad_output) {
  layer_norm_backward_task(scheduler, state, grad_output, nullptr, {false, true}, Task::Impl::kAssist,
                           "cs::compute::LayerNorm::backward_parameter");
}

Tensor LayerNorm::backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                           const ReadOnlyTensor &grad_output) {
  Tensor dx;
  if (ln_single_pass(scheduler, state, grad_output)) {
    dx = layer_norm_backward_task(scheduler, state, grad_output, nullptr, {true, true}, Task::Impl::kMain,
                                  "cs::compute::LayerNorm::backward");
  } else {
    backward_parameter(scheduler, state, grad_output);
    dx = backward_input(scheduler, state, grad_output);
  }
  ln_release(state);
  return dx;
}

Tensor LayerNorm::backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                           const ReadOnlyTensor &grad_output, const ReadOnlyTensor &grad_residual) {
  Tensor dx;
  if (ln_single_pass(scheduler, state, grad_output)) {
    dx = layer_norm_backward_task(scheduler, state, grad_output, &grad_residual, {true, true}, Task::Impl::kMain,
                                  "cs::compute::LayerNorm::backward");
  } else {
    backward_parameter(scheduler, state, grad_output);
    dx = layer_norm_backward_task(scheduler, state, grad_output, &grad_residual, {true, false}, Task::Impl::kMain,
                                  "cs::compute::LayerNorm::backward_input");
  }
  ln_release(state);
  return dx;
}

// ======================================================================================
// GeLU
// ======================================================================================
std::shared_ptr<GeLU::State> GeLU::init(const Scheduler &) { return std::make_shared<State>(); }

Tensor GeLU::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input) {
  Tensor output;
  state->backward.input = input;
  submit(scheduler, "cs::compute::GeLU::forward", Task::Impl::kMain, Task::Impl::kCompute, {output}, {input},
         [input, output](const FnTask &) {
           const at::Tensor x = input.impl()->tensor;
           if (x.is_cuda() && x.scalar_type() == at::kBFloat16 && fused_enabled() && x.is_contiguous()) {
             at::Tensor y = at::empty_like(x);
             check_kernel(kernels::gelu_forward(current_stream(), x.data_ptr(), y.data_ptr(), x.numel()), "gelu_forward");
             output.impl()->tensor = y;
           } else {
             output.impl()->tensor = at::gelu(x);
           }
         });
  return output;
}

Tensor GeLU::backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                      const ReadOnlyTensor &grad_output) {
  Tensor grad_input;
  submit(scheduler, "cs::compute::GeLU::backward", Task::Impl::kMain, Task::Impl::kCompute, {grad_input},
         {grad_output, state->backward.input}, [grad_output, x_h = state->backward.input, grad_input](const FnTask &) {
           const at::Tensor x = x_h.impl()->tensor;
           const at::Tensor dy = grad_output.impl()->tensor;
           if (x.is_cuda() && x.scalar_type() == at::kBFloat16 && dy.scalar_type() == at::kBFloat16 && fused_enabled() &&
               x.is_contiguous() && dy.is_contiguous()) {
             at::Tensor dx = at::empty_like(x);
             check_kernel(kernels::gelu_backward(current_stream(), dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel()),
                          "gelu_backward");
             grad_input.impl()->tensor = dx;
           } else {
             grad_input.impl()->tensor = at::gelu_backward(dy, cast_if(x, dy.scalar_type()));
           }
         });
  state->backward.input.reset();
  return grad_input;
}

// ======================================================================================
// Embedding
// ======================================================================================
OrderedDict<std::string, Tensor> Embedding::State::parameters() const {
  OrderedDict<std::string, Tensor> d;
  d.insert("weight", forward.weight);
  return d;
}
OrderedDict<std::string, Tensor> Embedding::State::gradients() const {
  OrderedDict<std::string, Tensor> d;
  d.insert("weight", forward.grad_weight);
  return d;
}
OrderedDict<std::string, module::State::Increment> Embedding::State::increments() const {
  OrderedDict<std::string, Increment> d;
  d.insert("weight", {forward.weight, forward.grad_weight});
  return d;
}
void Embedding::State::zero_grad() { module::clear_gradient(forward.grad_weight); }

std::shared_ptr<Embedding::State> Embedding::init(const Scheduler &scheduler, const Options &options) {
  CS_ASSERT_TRUE(!options.max_norm().has_value(), "Embedding max_norm is not supported");
  int64_t padding_idx = -1;
  if (options.padding_idx().has_value()) {
    padding_idx = *options.padding_idx();
    if (padding_idx < 0) padding_idx += options.num_embeddings();
    CS_ASSERT_TRUE(padding_idx >= 0 && padding_idx < options.num_embeddings(), "padding_idx out of range");
  }
  Tensor weight;
  TensorOptions topt{};
  topt = topt.device(options.device().value_or(scheduler.device())).dtype(options.dtype().value_or(at::kFloat));
  submit(scheduler, "cs::compute::Embedding::init", Task::Impl::kMain, Task::Impl::kCompute, {weight}, {},
         [weight, topt, n = options.num_embeddings(), d = options.embedding_dim(), padding_idx](const FnTask &) {
           weight.impl()->tensor = at::empty({n, d}, topt).normal_(0, 1);
           if (padding_idx >= 0) weight.impl()->tensor[padding_idx].zero_();
           ++weight.impl()->version;
         });
  return std::make_shared<State>(State::Forward{weight}, State::Backward{},
                                 State::Args{options.num_embeddings(), padding_idx, options.max_norm(),
                                             options.norm_type(), options.scale_grad_by_freq(), options.sparse()});
}

Tensor Embedding::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                          const ReadOnlyTensor &indices) {
  Tensor output;
  state->backward.indices = indices;
  const bool amp = scheduler.impl()->autocast_enabled;
  const at::ScalarType amp_dt = scheduler.impl()->autocast_dtype;
  submit(scheduler, "cs::compute::Embedding::forward", Task::Impl::kMain, Task::Impl::kCompute, {output},
         {indices, state->forward.weight}, [indices, w = state->forward.weight, output, amp, amp_dt](const FnTask &) {
           const at::Tensor idx = indices.impl()->tensor;
           const at::Tensor &wt = (amp && amp_dt == at::kBFloat16) ? kernel_view(w) : w.impl()->tensor;
           if (amp && amp_dt == at::kBFloat16 && wt.is_cuda() && fused_enabled() && idx.scalar_type() == at::kLong &&
               wt.size(1) % 8 == 0 && dtype_code(wt.scalar_type()) >= 0 && dtype_code(wt.scalar_type()) <= 1) {
             const at::Tensor ic = idx.contiguous();
             auto sizes = ic.sizes().vec();
             sizes.push_back(wt.size(1));
             at::Tensor out = at::empty(sizes, wt.options().dtype(at::kBFloat16));
             check_kernel(kernels::embedding_forward(current_stream(), ic.data_ptr<int64_t>(), wt.data_ptr(), nullptr,
                                                     dtype_code(wt.scalar_type()), out.data_ptr(), ic.numel(), 1,
                                                     wt.size(1), wt.size(0)),
                          "embedding_forward");
             output.impl()->tensor = out;
             return;
           }
           at::Tensor out = at::embedding(wt, idx);
           output.impl()->tensor = amp ? cast_if(out, amp_dt) : out;
         });
  return output;
}

namespace {
void embedding_backward_library(const at::Tensor &dy, const at::Tensor &idx, const Embedding::State::Args &args,
                                const Tensor &weight, const Tensor &grad_slot) {
  const at::ScalarType store = weight.impl()->tensor.scalar_type();
  at::Tensor g = at::embedding_backward(cast_if(dy, store == at::kDouble ? at::kDouble : at::kFloat), idx,
                                        args.num_embeddings, args.padding_idx, args.scale_grad_by_freq, false);
  store_grad(grad_slot, g, store);
}
}  // namespace

void Embedding::backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                         const ReadOnlyTensor &grad_output) {
  submit(scheduler, "cs::compute::Embedding::backward", Task::Impl::kAssist, Task::Impl::kCompute,
         {state->forward.grad_weight}, {grad_output, state->backward.indices, state->forward.weight},
         [grad_output, idx_h = state->backward.indices, w = state->forward.weight, gw = state->forward.grad_weight,
          args = state->args](const FnTask &) {
           const at::Tensor dy = grad_output.impl()->tensor.contiguous();
           const at::Tensor idx = idx_h.impl()->tensor.contiguous();
           const at::Tensor &wt = w.impl()->tensor;
           if (dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && fused_enabled() && wt.scalar_type() == at::kFloat &&
               idx.scalar_type() == at::kLong && !args.scale_grad_by_freq && wt.size(1) % 8 == 0) {
             auto &slot = *gw.impl();
             if (!slot.tensor.defined()) {
               slot.tensor = at::zeros_like(wt);
             } else if (slot.fresh) {
               slot.tensor.zero_();
             }
             slot.fresh = false;
             check_kernel(kernels::embedding_backward(current_stream(), idx.data_ptr<int64_t>(), dy.data_ptr(),
                                                      slot.tensor.data_ptr<float>(), nullptr, 0, idx.numel(), 1,
                                                      wt.size(1), wt.size(0), args.padding_idx),
                          "embedding_backward");
             return;
           }
           embedding_backward_library(dy, idx, args, w, gw);
         });
  state->backward.indices.reset();
}

Tensor Embedding::forward_token_position(const Scheduler &scheduler, const std::shared_ptr<State> &token,
                                         const std::shared_ptr<State> &position, const ReadOnlyTensor &indices) {
  Tensor output;
  token->backward.indices = indices;
  const bool amp = scheduler.impl()->autocast_enabled;
  const at::ScalarType amp_dt = scheduler.impl()->autocast_dtype;
  submit(scheduler, "cs::compute::Embedding::forward_token_position", Task::Impl::kMain, Task::Impl::kCompute, {output},
         {indices, token->forward.weight, position->forward.weight},
         [indices, wte = token->forward.weight, wpe = position->forward.weight, output, amp, amp_dt](const FnTask &) {
           const at::Tensor idx = indices.impl()->tensor.contiguous();
           const bool lp_tables = amp && amp_dt == at::kBFloat16 && kernel_view(wte).scalar_type() == kernel_view(wpe).scalar_type();
           const at::Tensor &te = lp_tables ? kernel_view(wte) : wte.impl()->tensor;
           const at::Tensor &pe = lp_tables ? kernel_view(wpe) : wpe.impl()->tensor;
           CS_ASSERT_TRUE(idx.dim() == 2, "token indices must be [batch, seq]");
           const int64_t T = idx.size(1);
           CS_ASSERT_TRUE(T <= pe.size(0), "sequence length ", T, " exceeds the position table (", pe.size(0), ")");
           if (amp && amp_dt == at::kBFloat16 && te.is_cuda() && fused_enabled() && idx.scalar_type() == at::kLong &&
               te.size(1) % 8 == 0 && te.scalar_type() == pe.scalar_type() && dtype_code(te.scalar_type()) >= 0 &&
               dtype_code(te.scalar_type()) <= 1) {
             at::Tensor out = at::empty({idx.size(0), T, te.size(1)}, te.options().dtype(at::kBFloat16));
             check_kernel(kernels::embedding_forward(current_stream(), idx.data_ptr<int64_t>(), te.data_ptr(),
                                                     pe.data_ptr(), dtype_code(te.scalar_type()), out.data_ptr(),
                                                     idx.numel(), T, te.size(1), te.size(0)),
                          "embedding_forward");
             output.impl()->tensor = out;
             return;
           }
           at::Tensor out = at::embedding(te, idx) + pe.narrow(0, 0, T).unsqueeze(0);
           output.impl()->tensor = amp ? cast_if(out, amp_dt) : out;
         });
  return output;
}

void Embedding::backward_token_position(const Scheduler &scheduler, const std::shared_ptr<State> &token,
                                        const std::shared_ptr<State> &position, const ReadOnlyTensor &grad_output) {
  submit(scheduler, "cs::compute::Embedding::backward_token_position", Task::Impl::kAssist, Task::Impl::kCompute,
         {token->forward.grad_weight, position->forward.grad_weight},
         {grad_output, token->backward.indices, token->forward.weight, position->forward.weight},
         [grad_output, idx_h = token->backward.indices, wte = token->forward.weight, wpe = position->forward.weight,
          gte = token->forward.grad_weight, gpe = position->forward.grad_weight, targs = token->args](const FnTask &) {
           const at::Tensor dy = grad_output.impl()->tensor.contiguous();
           const at::Tensor idx = idx_h.impl()->tensor.contiguous();
           const at::Tensor &te = wte.impl()->tensor;
           const at::Tensor &pe = wpe.impl()->tensor;
           const int64_t T = idx.size(1);
           if (dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && fused_enabled() && te.scalar_type() == at::kFloat &&
               pe.scalar_type() == at::kFloat && idx.scalar_type() == at::kLong && te.size(1) % 8 == 0) {
             auto &st = *gte.impl();
             auto &sp = *gpe.impl();
             if (!st.tensor.defined()) {
               st.tensor = at::zeros_like(te);
             } else if (st.fresh) {
               st.tensor.zero_();
             }
             st.fresh = false;
             int accumulate_pe = 1;
             if (!sp.tensor.defined()) {
               sp.tensor = at::zeros_like(pe);
             } else if (sp.fresh) {
               if (T < pe.size(0)) sp.tensor.zero_();
               accumulate_pe = T < pe.size(0) ? 1 : 0;
             }
             sp.fresh = false;
             check_kernel(kernels::embedding_backward(current_stream(), idx.data_ptr<int64_t>(), dy.data_ptr(),
                                                      st.tensor.data_ptr<float>(), sp.tensor.data_ptr<float>(),
                                                      accumulate_pe, idx.numel(), T, te.size(1), te.size(0),
                                                      targs.padding_idx),
                          "embedding_backward");
             return;
           }
           embedding_backward_library(dy, idx, targs, wte, gte);
           at::Tensor dpe = at::zeros_like(pe, pe.options().dtype(pe.scalar_type() == at::kDouble ? at::kDouble : at::kFloat));
           dpe.narrow(0, 0, T).copy_(at::sum(dy.to(dpe.scalar_type()), {0}));
           store_grad(gpe, dpe, pe.scalar_type());
         });
  token->backward.indices.reset();
}

// ======================================================================================
// CrossEntropy
// ======================================================================================
std::shared_ptr<CrossEntropy::State> CrossEntropy::init(const Scheduler &, const Options &options) {
  CS_ASSERT_TRUE(options.label_smoothing() == 0.0, "label smoothing is not supported");
  auto state = std::make_shared<State>();
  state->args = State::Args{options.reduction(), options.ignore_index(), options.label_smoothing()};
  return state;
}

Tensor CrossEntropy::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                             const ReadOnlyTensor &input, const ReadOnlyTensor &target) {
  Tensor loss, log_probs, total_weight;
  state->backward.log_probs = log_probs;
  state->backward.target = target;
  state->backward.total_weight = total_weight;
  state->backward.loss = loss;
  const bool amp = scheduler.impl()->autocast_enabled;
  submit(scheduler, "cs::compute::CrossEntropy::forward", Task::Impl::kMain, Task::Impl::kCompute,
         {loss, log_probs, total_weight}, {input, target, state->forward.weight},
         [input, target, weight = state->forward.weight, args = state->args, loss, log_probs, total_weight,
          amp](const FnTask &) {
           const at::Tensor &x = input.impl()->tensor;
           const bool low = x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16;
           const at::Tensor lp = at::log_softmax(x, 1, (amp || low) ? std::optional<at::ScalarType>{at::kFloat} : std::nullopt);
           std::optional<at::Tensor> wopt;
           if (weight.impl()->tensor.defined()) wopt = weight.impl()->tensor;
           auto [l, tw] = at::nll_loss_forward(lp, target.impl()->tensor, wopt, static_cast<int64_t>(args.reduction),
                                               args.ignore_index);
           loss.impl()->tensor = l;
           log_probs.impl()->tensor = lp;
           total_weight.impl()->tensor = tw;
           log_probs.impl()->companion = at::empty({0}, x.options());  // remembers the logits dtype
         });
  return loss;
}

Tensor CrossEntropy::backward(const Scheduler &scheduler, const std::shared_ptr<State> &state) {
  Tensor grad_input;
  submit(scheduler, "cs::compute::CrossEntropy::backward", Task::Impl::kMain, Task::Impl::kCompute, {grad_input},
         {state->backward.log_probs, state->backward.target, state->backward.total_weight, state->backward.loss},
         [lp_h = state->backward.log_probs, target = state->backward.target, tw = state->backward.total_weight,
          loss = state->backward.loss, weight = state->forward.weight, args = state->args, grad_input](const FnTask &) {
           const at::Tensor &lp = lp_h.impl()->tensor;
           std::optional<at::Tensor> wopt;
           if (weight.impl()->tensor.defined()) wopt = weight.impl()->tensor;
           at::Tensor seed = args.reduction == Reduction::kNone ? at::ones_like(loss.impl()->tensor)
                                                               : at::ones_like(loss.impl()->tensor);
           at::Tensor dlp = at::nll_loss_backward(seed, lp, target.impl()->tensor, wopt,
                                                  static_cast<int64_t>(args.reduction), args.ignore_index,
                                                  tw.impl()->tensor);
           at::Tensor dx = at::_log_softmax_backward_data(dlp, lp, 1, lp.scalar_type());
           const at::Tensor &tag = lp_h.impl()->companion;
           grad_input.impl()->tensor = tag.defined() ? cast_if(dx, tag.scalar_type()) : dx;
         });
  state->backward.log_probs.reset();
  state->backward.target.reset();
  state->backward.total_weight.reset();
  state->backward.loss.reset();
  return grad_input;
}

// ======================================================================================
// LinearCrossEntropy (fused classifier + loss)
// ======================================================================================
std::shared_ptr<LinearCrossEntropy::State> LinearCrossEntropy::init(const Scheduler &,
                                                                    const std::shared_ptr<Linear::State> &linear,
                                                                    int64_t valid_classes, int64_t ignore_index) {
  CS_ASSERT_TRUE(!linear->args.bias, "LinearCrossEntropy expects a classifier without bias");
  auto state = std::make_shared<State>();
  state->linear = linear;
  state->valid_classes = valid_classes;
  state->ignore_index = ignore_index;
  return state;
}

Tensor LinearCrossEntropy::forward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                   const ReadOnlyTensor &input, const ReadOnlyTensor &target) {
  Tensor loss, logits, lse;
  state->backward.input = input;
  state->backward.target = target;
  state->backward.logits = logits;
  state->backward.lse = lse;
  const auto &w = state->linear->forward.weight;
  const at::ScalarType amp_dt = matmul_dtype(scheduler, input, w, Tensor{});
  submit(scheduler, "cs::compute::LinearCrossEntropy::forward", Task::Impl::kMain, Task::Impl::kCompute,
         {loss, logits, lse}, {input, target, w},
         [input, target, w, amp_dt, loss, logits, lse, valid = state->valid_classes,
          ignore = state->ignore_index](const FnTask &task) {
           const at::Tensor &x = input.impl()->tensor;
           const at::ScalarType dt = amp_dt == at::ScalarType::Undefined ? x.scalar_type() : amp_dt;
           const at::Tensor x2 = as2d(cast_if(x, dt));
           const at::Tensor wc = working_copy(w, dt);
           const at::Tensor tgt = target.impl()->tensor.reshape({-1}).contiguous();
           const int64_t rows = x2.size(0), V = wc.size(0);
           const int64_t n_valid = valid > 0 ? valid : V;
           if (x2.is_cuda() && dt == at::kBFloat16 && fused_enabled() && tgt.scalar_type() == at::kLong) {
             const int64_t n_tiles = kernels::gemm_ce_stat_tiles(V);
             at::Tensor lg = at::empty({rows, V}, x2.options());
             at::Tensor stats = at::empty({rows, n_tiles, 2}, x2.options().dtype(at::kFloat));
             kernels::GemmArgs g{};
             g.a = x2.data_ptr();
             g.b = wc.data_ptr();
             g.d = lg.data_ptr();
             g.stats = stats.data_ptr<float>();
             g.m = rows;
             g.n = V;
             g.k = x2.size(1);
             g.lda = g.k;
             g.ldb = g.k;
             g.ldd = V;
             g.layout = kernels::kTN;
             g.epilogue = kernels::kEpiCrossEntropy;
             g.n_valid = n_valid;
             if (fused_gemm(g)) {
               task.intermediate().push_back(stats);
               at::Tensor l = at::empty({}, x2.options().dtype(at::kFloat));
               at::Tensor ls = at::empty({rows + 1}, x2.options().dtype(at::kFloat));  // [rows] lse + valid-row count
               check_kernel(kernels::cross_entropy_finalize(current_stream(), stats.data_ptr<float>(), n_tiles,
                                                            lg.data_ptr(), V, tgt.data_ptr<int64_t>(),
                                                            ls.data_ptr<float>(), l.data_ptr<float>(),
                                                            ls.data_ptr<float>() + rows, rows, ignore),
                            "cross_entropy_finalize");
               loss.impl()->tensor = l;
               logits.impl()->tensor = lg;
               lse.impl()->tensor = ls;
               return;
             }
           }
           // Library path: materialise logits, fp32 log-softmax.
           at::Tensor lg = at::linear(x2, wc);
           at::Tensor lgv = n_valid < V ? lg.narrow(1, 0, n_valid) : lg;
           at::Tensor lsev = at::logsumexp(lgv.to(x2.scalar_type() == at::kDouble ? at::kDouble : at::kFloat), {1});
           at::Tensor logp = at::log_softmax(lgv, 1, x2.scalar_type() == at::kDouble ? at::kDouble : at::kFloat);
           auto [l, tw] = at::nll_loss_forward(logp, tgt, std::nullopt, 1, ignore);
           loss.impl()->tensor = l;
           logits.impl()->tensor = lg;
           lse.impl()->tensor = at::cat({lsev.to(at::kFloat), tw.reshape({1}).to(at::kFloat)});
         });
  return loss;
}

Tensor LinearCrossEntropy::backward(const Scheduler &scheduler, const std::shared_ptr<State> &state) {
  Tensor grad_input, dlogits;
  const auto &lin = state->linear;
  // 1) logits -> dlogits (in place on the fused path)
  submit(scheduler, "cs::compute::LinearCrossEntropy::backward_logits", Task::Impl::kMain, Task::Impl::kCompute,
         {dlogits}, {state->backward.logits, state->backward.lse, state->backward.target},
         [lg_h = state->backward.logits, lse_h = state->backward.lse, target = state->backward.target, dlogits,
          valid = state->valid_classes, ignore = state->ignore_index](const FnTask &) {
           at::Tensor lg = lg_h.impl()->tensor;
           const at::Tensor &ls = lse_h.impl()->tensor;
           const at::Tensor tgt = target.impl()->tensor.reshape({-1}).contiguous();
           const int64_t rows = lg.size(0), V = lg.size(1);
           const int64_t n_valid = valid > 0 ? valid : V;
           if (lg.is_cuda() && lg.scalar_type() == at::kBFloat16 && fused_enabled() && tgt.scalar_type() == at::kLong) {
             check_kernel(kernels::cross_entropy_backward_inplace(current_stream(), lg.data_ptr(), V,
                                                                  ls.data_ptr<float>(), tgt.data_ptr<int64_t>(),
                                                                  ls.data_ptr<float>() + rows, 1.0f, rows, V, n_valid,
                                                                  ignore),
                          "cross_entropy_backward_inplace");
             dlogits.impl()->tensor = lg;
             return;
           }
           const at::ScalarType ct = lg.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
           at::Tensor p = at::exp(lg.to(ct) - ls.narrow(0, 0, rows).to(ct).unsqueeze(1));
           if (n_valid < V) p.narrow(1, n_valid, V - n_valid).zero_();
           at::Tensor keep = tgt.ne(ignore);
           at::Tensor safe_t = at::where(keep, tgt, at::zeros_like(tgt));
           p.scatter_add_(1, safe_t.unsqueeze(1), -keep.to(ct).unsqueeze(1));
           p.mul_(keep.to(ct).unsqueeze(1));
           p.div_(ls.narrow(0, rows, 1).to(ct));
           dlogits.impl()->tensor = p.to(lg.scalar_type());
         });
  // 2) d(input) on the main stream, 3) classifier weight gradient on the assist stream
  submit(scheduler, "cs::compute::LinearCrossEntropy::backward_input", Task::Impl::kMain, Task::Impl::kCompute,
         {grad_input}, {dlogits, lin->forward.weight, state->backward.input},
         [dlogits, w = lin->forward.weight, x_h = state->backward.input, grad_input](const FnTask &) {
           const at::Tensor &dl = dlogits.impl()->tensor;
           at::Tensor dx = linear_dgrad(dl, w, dl.scalar_type(), nullptr);
           grad_input.impl()->tensor = dx.view(x_h.impl()->tensor.sizes());
         });
  submit(scheduler, "cs::compute::LinearCrossEntropy::backward_parameter", Task::Impl::kAssist, Task::Impl::kCompute,
         {lin->forward.grad_weight}, {dlogits, state->backward.input, lin->forward.weight},
         [dlogits, x_h = state->backward.input, w = lin->forward.weight, gw = lin->forward.grad_weight](const FnTask &) {
           const at::Tensor &dl = dlogits.impl()->tensor;
           linear_wgrad(dl, x_h.impl()->tensor, dl.scalar_type(), w, gw);
         });
  state->backward.input.reset();
  state->backward.target.reset();
  state->backward.logits.reset();
  state->backward.lse.reset();
  return grad_input;
}
}  // namespace cs::compute
