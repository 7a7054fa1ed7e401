// SPDX-License-Identifier: Apache-2.0
// AdamW / AmpAdamW functional ops and module::AdamW. See cs/optimizer.h for the parity map.
#include "cs/optimizer.h"

#include <algorithm>
#include <cmath>

#include "cs/compute.h"
#include "op_common.h"

namespace cs::optimizer {
using namespace compute::detail;

namespace {
AdamW::State::Options to_state_options(const AdamW::Options &o) {
  AdamW::State::Options s;
  s.lr = o.lr();
  s.beta1 = o.beta1();
  s.beta2 = o.beta2();
  s.eps = o.eps();
  s.weight_decay = o.weight_decay();
  s.amsgrad = o.amsgrad();
  s.t = o.t();
  return s;
}

// The update on one tensor (any device/dtype). Refreshes the working copies of `w`.
void adamw_update(const at::Tensor &w, const at::Tensor &g_in, const at::Tensor &m, const at::Tensor &v,
                  const at::Tensor &v_max, const AdamW::State::Options &o, int64_t t, const at::Tensor &clip,
                  ReadOnlyTensor::Impl *w_impl, const at::Tensor &lp_override) {
  const double bc1 = 1.0 - std::pow(o.beta1, static_cast<double>(t));
  const double bc2 = 1.0 - std::pow(o.beta2, static_cast<double>(t));
  at::Tensor lp = lp_override.defined() ? lp_override : (w_impl ? w_impl->lp : at::Tensor{});
  const int pcode = dtype_code(w.scalar_type());
  const int gcode = dtype_code(g_in.scalar_type());
  const bool lp_ok = !lp.defined() || (lp.scalar_type() == at::kBFloat16 && lp.is_contiguous());
  if (w.is_cuda() && fused_enabled() && pcode >= 0 && gcode >= 0 && w.is_contiguous() && g_in.is_contiguous() &&
      m.is_contiguous() && v.is_contiguous() && lp_ok && m.scalar_type() == w.scalar_type()) {
    kernels::AdamWArgs a{};
    a.param = w.data_ptr();
    a.grad = g_in.data_ptr();
    a.exp_avg = m.data_ptr();
    a.exp_avg_sq = v.data_ptr();
    a.max_exp_avg_sq = o.amsgrad ? v_max.data_ptr() : nullptr;
    a.lp = lp.defined() ? lp.data_ptr() : nullptr;
    a.n = w.numel();
    a.param_dtype = pcode;
    a.grad_dtype = gcode;
    a.lr = static_cast<float>(o.lr);
    a.beta1 = static_cast<float>(o.beta1);
    a.beta2 = static_cast<float>(o.beta2);
    a.eps = static_cast<float>(o.eps);
    a.weight_decay = static_cast<float>(o.weight_decay);
    a.inv_bias_correction1 = static_cast<float>(1.0 / bc1);
    a.inv_bias_correction2 = static_cast<float>(1.0 / bc2);
    a.grad_scale = static_cast<float>(o.grad_scale);
    a.clip_coef = clip.defined() ? clip.data_ptr<float>() : nullptr;
    check_kernel(kernels::adamw_step(current_stream(), a), "adamw_step");
  } else {
    // ATen path: math in fp32 (fp64 for double parameters), states kept in their own dtype.
    const at::ScalarType ct = w.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
    at::Tensor g = g_in.to(ct);
    if (o.grad_scale != 1.0) g = g * o.grad_scale;
    if (clip.defined()) g = g * clip.to(ct);
    at::Tensor wf = w.to(ct), mf = m.to(ct), vf = v.to(ct);
    wf = wf - o.lr * o.weight_decay * wf;
    mf = o.beta1 * mf + (1 - o.beta1) * g;
    vf = o.beta2 * vf + (1 - o.beta2) * g * g;
    at::Tensor m_hat = mf / bc1;
    at::Tensor v_hat = vf / bc2;
    if (o.amsgrad) {
      at::Tensor vm = at::maximum(v_max.to(ct), v_hat);
      v_max.copy_(vm);
      v_hat = vm;
    }
    wf = wf - o.lr * m_hat / (at::sqrt(v_hat) + o.eps);
    w.copy_(wf);
    m.copy_(mf);
    v.copy_(vf);
    if (lp.defined()) lp.copy_(w);
  }
  if (w_impl) {
    ++w_impl->version;
    if (w_impl->lp.defined()) w_impl->lp_version = w_impl->version;
  }
}
}  // namespace

std::shared_ptr<AdamW::State> AdamW::init(const Scheduler &scheduler, const ReadOnlyTensor &parameter,
                                          const Options &options) {
  Tensor m, v, v_max;
  std::vector<Tensor> outs{m, v};
  if (options.amsgrad()) outs.push_back(v_max);
  submit(scheduler, "cs::optimizer::AdamW::init", Task::Impl::kAssist, Task::Impl::kCompute, outs, {parameter},
         [parameter, m, v, v_max, amsgrad = options.amsgrad()](const FnTask &) {
           const at::Tensor &p = parameter.impl()->tensor;
           m.impl()->tensor = at::zeros_like(p);
           v.impl()->tensor = at::zeros_like(p);
           if (amsgrad) v_max.impl()->tensor = at::zeros_like(p);
         });
  return std::make_shared<State>(State::Tensors{m, v, v_max}, to_state_options(options));
}

void AdamW::step(const Scheduler &scheduler, const std::shared_ptr<State> &state, const Tensor &w,
                 const ReadOnlyTensor &dw) {
  if (!dw.defined()) {
    CS_WARN_TRUE(false, "AdamW::step got an undefined gradient; the parameter is left unchanged");
    return;
  }
  const int64_t t = ++state->options.t;
  std::vector<Tensor> outs{w, state->tensors.m, state->tensors.v};
  if (state->options.amsgrad) outs.push_back(state->tensors.v_max);
  std::vector<ReadOnlyTensor> ins{dw};
  if (state->clip_coef.defined()) ins.push_back(state->clip_coef);
  submit(scheduler, "cs::optimizer::AdamW::step", Task::Impl::kAssist, Task::Impl::kCompute, outs, ins,
         [w, dw, tensors = state->tensors, o = state->options, t, clip = state->clip_coef](const FnTask &) {
           adamw_update(w.impl()->tensor, dw.impl()->tensor, tensors.m.impl()->tensor, tensors.v.impl()->tensor,
                        tensors.v_max.impl()->tensor, o, t, clip.impl()->tensor, w.impl().get(), at::Tensor{});
         });
}

std::shared_ptr<AdamW::State> AmpAdamW::init(const Scheduler &scheduler, const ReadOnlyTensor &parameterFp32,
                                             const Options &options) {
  return AdamW::init(scheduler, parameterFp32, options);
}

void AmpAdamW::step(const Scheduler &scheduler, const std::shared_ptr<State> &state, const Tensor &w,
                    const Tensor &wFp32, const ReadOnlyTensor &dw) {
  if (!dw.defined()) {
    CS_WARN_TRUE(false, "AmpAdamW::step got an undefined gradient; the parameter is left unchanged");
    return;
  }
  const int64_t t = ++state->options.t;
  std::vector<Tensor> outs{w, wFp32, state->tensors.m, state->tensors.v};
  if (state->options.amsgrad) outs.push_back(state->tensors.v_max);
  submit(scheduler, "cs::optimizer::AmpAdamW::step", Task::Impl::kAssist, Task::Impl::kCompute, outs, {dw},
         [w, wFp32, dw, tensors = state->tensors, o = state->options, t, clip = state->clip_coef](const FnTask &) {
           const at::Tensor &low = w.impl()->tensor;
           const bool kernel_lp = low.scalar_type() == at::kBFloat16 && low.is_contiguous();
           adamw_update(wFp32.impl()->tensor, dw.impl()->tensor, tensors.m.impl()->tensor, tensors.v.impl()->tensor,
                        tensors.v_max.impl()->tensor, o, t, clip.impl()->tensor, wFp32.impl().get(),
                        kernel_lp ? low : at::Tensor{});
           if (!kernel_lp) low.copy_(wFp32.impl()->tensor);
           ++w.impl()->version;
         });
}
}  // namespace cs::optimizer

namespace cs::module {
using OptAdamW = optimizer::AdamW;

AdamWImpl::AdamWImpl(const Scheduler &scheduler, const std::shared_ptr<Module> &module, const Options &options) {
  bind(module);
  build(scheduler, *module, options);
}
AdamWImpl::AdamWImpl(const Scheduler &scheduler, const Module &module, const Options &options) {
  bind(&module);
  build(scheduler, module, options);
}
AdamWImpl::AdamWImpl(const Scheduler &scheduler, const Module &module, const std::shared_ptr<FlatParameters> &flat,
                     const Options &options)
    : flat_{flat} {
  bind(&module);
  build(scheduler, module, options);
}

void AdamWImpl::build(const Scheduler &scheduler, const Module &module, const Options &options) {
  if (!flat_) {
    for (auto &item : module.named_parameters()) {
      states_.insert(item.first, OptAdamW::init(scheduler, item.second, options));
    }
    return;
  }
  // One pair of flat moment buffers; the per-parameter states are views into them so the
  // named-state interface (and checkpoints) look the same as in the per-tensor layout.
  flat_state_ = OptAdamW::init(scheduler, flat_->params, options);
  auto named = module.named_parameters();
  for (auto &slot : flat_->slots) {
    Tensor m, v, vmax;
    std::vector<Tensor> outs{m, v};
    if (options.amsgrad()) outs.push_back(vmax);
    auto sizes = named[slot.key].sizes().vec();
    submit(scheduler, "cs::module::AdamW::view_state", Task::Impl::kAssist, Task::Impl::kCompute, outs,
           {flat_state_->tensors.m, flat_state_->tensors.v, flat_state_->tensors.v_max},
           [fs = flat_state_, m, v, vmax, slot, sizes, amsgrad = options.amsgrad()](const FnTask &) {
             m.impl()->tensor = fs->tensors.m.impl()->tensor.narrow(0, slot.offset, slot.numel).view(sizes);
             v.impl()->tensor = fs->tensors.v.impl()->tensor.narrow(0, slot.offset, slot.numel).view(sizes);
             if (amsgrad)
               vmax.impl()->tensor = fs->tensors.v_max.impl()->tensor.narrow(0, slot.offset, slot.numel).view(sizes);
           });
    auto st = std::make_shared<OptAdamW::State>(OptAdamW::State::Tensors{m, v, vmax}, flat_state_->options);
    states_.insert(slot.key, st);
  }
}

void AdamWImpl::set_grad_scale(double scale) {
  if (flat_state_) flat_state_->options.grad_scale = scale;
  for (auto &s : states_) std::dynamic_pointer_cast<OptAdamW::State>(s.second)->options.grad_scale = scale;
}
void AdamWImpl::set_clip_coefficient(const Tensor &coef) {
  if (flat_state_) flat_state_->clip_coef = coef;
  for (auto &s : states_) std::dynamic_pointer_cast<OptAdamW::State>(s.second)->clip_coef = coef;
}

int64_t AdamWImpl::step_count() const {
  if (flat_state_) return flat_state_->options.t;
  for (auto &s : states_) return std::dynamic_pointer_cast<OptAdamW::State>(s.second)->options.t;
  return 0;
}
void AdamWImpl::set_step_count(int64_t t) {
  if (flat_state_) flat_state_->options.t = t;
  for (auto &s : states_) std::dynamic_pointer_cast<OptAdamW::State>(s.second)->options.t = t;
}

OrderedDict<std::string, Tensor> AdamWImpl::named_state_tensors() const {
  OrderedDict<std::string, Tensor> out;
  for (auto &s : states_) {
    auto st = std::dynamic_pointer_cast<OptAdamW::State>(s.second);
    out.insert(s.first + ".m", st->tensors.m);
    out.insert(s.first + ".v", st->tensors.v);
    if (st->options.amsgrad) out.insert(s.first + ".v_max", st->tensors.v_max);
  }
  return out;
}

void AdamWImpl::open_step() {
  step_open_ = true;
  for (auto &s : states_) {  // set_lr() touches the per-parameter views; the flat state follows
    flat_state_->options.lr = s.second->get_lr();
    break;
  }
  ++flat_state_->options.t;
  for (auto &s : states_) std::dynamic_pointer_cast<OptAdamW::State>(s.second)->options.t = flat_state_->options.t;
  if (slot_params_.empty()) {
    const Module *m = model();
    CS_ASSERT_TRUE(m != nullptr, "the optimised module is gone");
    auto named = m->named_parameters();
    for (size_t i = 0; i < flat_->slots.size(); ++i) {
      slot_params_.push_back(named[flat_->slots[i].key]);
      slot_of_grad_.emplace(flat_->grad_handles[i].impl().get(), i);
    }
  }
  slot_done_.assign(flat_->slots.size(), 0);
}

void AdamWImpl::step_partial(const Scheduler &scheduler, const std::vector<Tensor> &gradients, Task::Impl::Priority priority) {
  CS_ASSERT_TRUE(flat_ != nullptr, "step_partial needs an optimizer over flat arenas");
  if (flat_state_->clip_coef.defined()) return;
  if (!step_open_) open_step();
  std::vector<size_t> picked;
  for (auto &g : gradients) {
    auto it = slot_of_grad_.find(g.impl().get());
    if (it == slot_of_grad_.end() || slot_done_[it->second]) continue;
    slot_done_[it->second] = 1;
    picked.push_back(it->second);
  }
  if (picked.empty()) return;
  std::sort(picked.begin(), picked.end());
  // neighbouring slots are contiguous in the arenas (padding included): one launch per run of slots
  struct Range {
    int64_t begin, end;
  };
  std::vector<Range> ranges;
  std::vector<Tensor> outs;
  std::vector<ReadOnlyTensor> ins;
  auto slot_end = [&](size_t i) {
    return i + 1 < flat_->slots.size() ? flat_->slots[i + 1].offset : flat_->total;
  };
  for (size_t k = 0; k < picked.size(); ++k) {
    const size_t i = picked[k];
    if (k > 0 && picked[k - 1] + 1 == i)
      ranges.back().end = slot_end(i);
    else
      ranges.push_back({flat_->slots[i].offset, slot_end(i)});
    outs.push_back(slot_params_[i]);
    ins.push_back(flat_->grad_handles[i]);
  }
  submit(scheduler, "cs::module::AdamW::step_partial", priority, Task::Impl::kCompute, outs, ins,
         [flat = flat_, fs = flat_state_, o = flat_state_->options, ranges, outs, handles = ins](const FnTask &) {
           const at::Tensor &P = flat->params.impl()->tensor, &G = flat->grads.impl()->tensor;
           const at::Tensor &M = fs->tensors.m.impl()->tensor, &V = fs->tensors.v.impl()->tensor;
           const at::Tensor &VM = fs->tensors.v_max.impl()->tensor;
           const at::Tensor L = flat->lp.defined() ? flat->lp.impl()->tensor : at::Tensor{};
           for (auto &h : handles)  // a slot nobody wrote this step must not contribute stale values
             if (h.impl()->fresh && h.impl()->tensor.defined()) const_cast<at::Tensor &>(h.impl()->tensor).zero_();
           for (auto &r : ranges) {
             const int64_t n = r.end - r.begin;
             optimizer::adamw_update(P.narrow(0, r.begin, n), G.narrow(0, r.begin, n), M.narrow(0, r.begin, n), V.narrow(0, r.begin, n),
                                     o.amsgrad ? VM.narrow(0, r.begin, n) : at::Tensor{}, o, o.t, at::Tensor{}, nullptr,
                                     L.defined() ? L.narrow(0, r.begin, n) : at::Tensor{});
           }
           for (auto &p : outs) {
             auto &impl = *p.impl();
             ++impl.version;
             if (impl.lp.defined()) impl.lp_version = impl.version;  // written by the kernel
             if (impl.lp_t.defined()) compute::working_copy_transposed(p, impl.lp_t.scalar_type());
           }
         });
}

void AdamWImpl::step(const Scheduler &scheduler) {
  const Module *m = model();
  CS_ASSERT_TRUE(m != nullptr, "the optimised module is gone");
  if (flat_ && step_open_) {
    // Buckets were updated while the backward pass ran: update what is left, then tie the arena handles
    // to everything that touched them.
    std::vector<Tensor> rest;
    for (size_t i = 0; i < flat_->slots.size(); ++i)
      if (!slot_done_[i]) rest.push_back(flat_->grad_handles[i]);
    step_partial(scheduler, rest, Task::Impl::kAssist);
    step_open_ = false;
    std::vector<ReadOnlyTensor> ins(slot_params_.begin(), slot_params_.end());
    std::vector<Tensor> outs{flat_->params, flat_state_->tensors.m, flat_state_->tensors.v};
    if (flat_->lp.defined()) outs.push_back(flat_->lp);
    submit(scheduler, "cs::module::AdamW::close_step", Task::Impl::kAssist, Task::Impl::kCompute, outs, ins, [](const FnTask &) {});
    return;
  }
  if (flat_) {
    // Keep the learning rate of the flat state in sync with set_lr() (which touches the views).
    for (auto &s : states_) {
      flat_state_->options.lr = s.second->get_lr();
      break;
    }
    // Low-precision copies live in the arena as well: hand them to the kernel through the
    // parameter handle, then refresh the transposed copies of the matrices.
    auto &pimpl = *flat_->params.impl();
    if (flat_->lp.defined()) {
      pimpl.lp = flat_->lp.impl()->tensor;
    }
    // Gradients are written through the per-parameter views (by backward on the assist stream and
    // by collectives on the comm stream); joining them here orders the update after all of them.
    {
      std::vector<ReadOnlyTensor> writers(flat_->grad_handles.begin(), flat_->grad_handles.end());
      submit(scheduler, "cs::module::AdamW::join_gradients", Task::Impl::kAssist, Task::Impl::kCompute, {flat_->grads},
             writers, [handles = flat_->grad_handles](const FnTask &) {
               // a slot nobody wrote this step must not contribute stale values
               for (auto &h : handles)
                 if (h.impl()->fresh && h.impl()->tensor.defined()) h.impl()->tensor.zero_();
             });
    }
    OptAdamW::step(scheduler, flat_state_, flat_->params, flat_->grads);
    for (auto &s : states_) std::dynamic_pointer_cast<OptAdamW::State>(s.second)->options.t = flat_state_->options.t;
    auto named = m->named_parameters();
    std::vector<Tensor> touched;
    for (auto &slot : flat_->slots) touched.push_back(named[slot.key]);
    std::vector<Tensor> outs = touched;
    submit(scheduler, "cs::module::AdamW::refresh_copies", Task::Impl::kAssist, Task::Impl::kCompute, outs,
           {flat_->params}, [touched](const FnTask &) {
             for (auto &p : touched) {
               auto &impl = *p.impl();
               ++impl.version;
               if (impl.lp.defined()) impl.lp_version = impl.version;  // written by the flat kernel
               if (impl.lp_t.defined()) compute::working_copy_transposed(p, impl.lp_t.scalar_type());
             }
           });
    return;
  }
  auto increments = m->named_increments();
  for (auto &s : states_) {
    auto *inc = increments.find(s.first);
    CS_ASSERT_TRUE(inc != nullptr, "parameter `", s.first, "` vanished from the module");
    OptAdamW::step(scheduler, std::dynamic_pointer_cast<OptAdamW::State>(s.second), inc->parameter, inc->gradient);
  }
}
}  // namespace cs::module
