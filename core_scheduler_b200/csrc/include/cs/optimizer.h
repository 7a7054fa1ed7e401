// SPDX-License-Identifier: Apache-2.0
// Functional optimizers and their module wrappers.
//
// Capability parity (reference project paths): include/optimizer/adamw.h:31-74,
// src/optimizer/adamw.cpp:29-170, src/optimizer/adamw.cu:25-151 (AdamW / AMSGrad update rule),
// include/optimizer/amp_adamw.h:29-43 (declared there without a body; implemented here),
// include/module/adamw.h + src/module/adamw.cpp:20-39 (one state per named parameter).
//
// Differences: bias corrections use a per-state step counter that advances once per step()
// call; the CUDA path is one vectorised launch per tensor, or a single launch for a whole
// model when its parameters live in flat arenas, and it refreshes the bf16 working copies
// in the same pass.
#pragma once
#include <unordered_map>

#include "cs/core.h"
#include "cs/module.h"

namespace cs::optimizer {
struct CS_API AdamW {
  struct State : module::OptimizerState {
    struct Tensors {
      Tensor m;
      Tensor v;
      Tensor v_max{};
    } tensors;
    struct Options {
      mutable double lr = 1e-3;
      double beta1 = 0.9;
      double beta2 = 0.999;
      double eps = 1e-8;
      double weight_decay = 1e-2;
      bool amsgrad = false;
      int64_t t = 0;
      double grad_scale = 1.0;  // extension: gradients are multiplied by this inside the kernel
    } options;
    Tensor clip_coef{};  // extension: optional device scalar multiplied into the gradient
    State(const Tensors &tensors, const Options &options) : tensors{tensors}, options{options} {}
    void set_lr(double lr) const override { options.lr = lr; }
    [[nodiscard]] double get_lr() const override { return options.lr; }
  };
  struct Options {
    Options() {}
    CS_ARG(double, lr) = 1e-3;
    CS_ARG(double, beta1) = 0.9;
    CS_ARG(double, beta2) = 0.999;
    CS_ARG(double, eps) = 1e-8;
    CS_ARG(double, weight_decay) = 1e-2;
    CS_ARG(bool, amsgrad) = false;
    CS_ARG(int64_t, t) = 0;
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler, const ReadOnlyTensor &parameter,
                                     const Options &options);
  static void step(const Scheduler &scheduler, const std::shared_ptr<State> &state, const Tensor &w,
                   const ReadOnlyTensor &dw);
};

// Mixed-precision AdamW: fp32 master weights and moments, low-precision working weights that
// the forward/backward passes read.
struct CS_API AmpAdamW : AdamW {
  static std::shared_ptr<State> init(const Scheduler &scheduler, const ReadOnlyTensor &parameterFp32,
                                     const Options &options);
  static void step(const Scheduler &scheduler, const std::shared_ptr<State> &state, const Tensor &w,
                   const Tensor &wFp32, const ReadOnlyTensor &dw);
};
}  // namespace cs::optimizer

namespace cs::module {
struct CS_API AdamWImpl : OptimizerModule {
  using Options = optimizer::AdamW::Options;
  AdamWImpl(const Scheduler &scheduler, const std::shared_ptr<Module> &module, const Options &options);
  AdamWImpl(const Scheduler &scheduler, const Module &module, const Options &options);
  template <typename ImplT>
  AdamWImpl(const Scheduler &scheduler, const ModuleHolder<ImplT> &holder, const Options &options)
      : AdamWImpl(scheduler, std::static_pointer_cast<Module>(holder.ptr()), options) {}
  // extension: whole-model update over flat arenas in one kernel launch.
  AdamWImpl(const Scheduler &scheduler, const Module &module, const std::shared_ptr<FlatParameters> &flat,
            const Options &options);
  void step(const Scheduler &scheduler) override;
  // extension (flat arenas only): updates just the parameters whose gradient handles are given, as one launch
  // per contiguous arena range, on the stream class `priority`. The first call after step() opens a new
  // optimizer step (advances the step counter once); step() then updates whatever is left and closes it.
  // Meant to be driven from communication::AllReduceBucket::on_reduced so that the update of a bucket's
  // parameters overlaps the rest of the backward pass. Does nothing while a clip coefficient is set (the
  // global gradient norm is only known after the whole backward pass): step() then updates everything.
  void step_partial(const Scheduler &scheduler, const std::vector<Tensor> &gradients, Task::Impl::Priority priority);
  [[nodiscard]] OrderedDict<std::string, Tensor> named_state_tensors() const override;
  [[nodiscard]] int64_t step_count() const override;
  void set_step_count(int64_t t) override;
  // extension: multiply gradients by `scale` (e.g. 1/world) and by a device-side clip factor.
  void set_grad_scale(double scale);
  void set_clip_coefficient(const Tensor &coef);
  [[nodiscard]] const std::shared_ptr<FlatParameters> &flat() const { return flat_; }
  [[nodiscard]] const std::shared_ptr<optimizer::AdamW::State> &flat_state() const { return flat_state_; }

 private:
  void build(const Scheduler &scheduler, const Module &module, const Options &options);
  void open_step();
  std::shared_ptr<FlatParameters> flat_;
  std::shared_ptr<optimizer::AdamW::State> flat_state_;
  // step_partial bookkeeping: slot index of every gradient handle, which slots the open step has updated
  std::unordered_map<const void *, size_t> slot_of_grad_;
  std::vector<Tensor> slot_params_;
  std::vector<char> slot_done_;
  bool step_open_{false};
};
CS_MODULE(AdamW);
}  // namespace cs::module
