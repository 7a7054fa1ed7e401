// SPDX-License-Identifier: Apache-2.0
// Stateful wrappers of the parameter-owning ops (what model code is written against).
// Capability parity (reference project paths): include/module/{linear,gelu_linear,layer_norm,
// embedding}.h and src/module/*.cpp: forward / backward (parameter gradient task and input
// gradient task) / backward_input / backward_parameter / state().
#pragma once
#include "cs/compute.h"
#include "cs/module.h"

namespace cs::module {
struct CS_API LinearImpl : Module {
  using Options = compute::Linear::Options;
  LinearImpl(const Scheduler &scheduler, const Options &options);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &input) const;
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &input, const ReadOnlyTensor &residual) const;
  // input gradient on the main stream first, then the weight gradient on the assist stream
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  Tensor backward_input(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  void backward_parameter(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  [[nodiscard]] std::shared_ptr<compute::Linear::State> state() const { return state_.lock(); }

 private:
  std::weak_ptr<compute::Linear::State> state_;
};
CS_MODULE(Linear);

struct CS_API GeluLinearImpl : Module {
  using Options = compute::GeluLinear::Options;
  GeluLinearImpl(const Scheduler &scheduler, const Options &options);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &input) const;
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &input, const ReadOnlyTensor &residual) const;
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  Tensor backward_input(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  void backward_parameter(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  [[nodiscard]] std::shared_ptr<compute::GeluLinear::State> state() const { return state_.lock(); }

 private:
  std::weak_ptr<compute::GeluLinear::State> state_;
};
CS_MODULE(GeluLinear);

struct CS_API LayerNormImpl : Module {
  using Options = compute::LayerNorm::Options;
  LayerNormImpl(const Scheduler &scheduler, const Options &options);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &input) const;
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output,
                  const ReadOnlyTensor &grad_residual) const;
  [[nodiscard]] std::shared_ptr<compute::LayerNorm::State> state() const { return state_.lock(); }

 private:
  std::weak_ptr<compute::LayerNorm::State> state_;
};
CS_MODULE(LayerNorm);

struct CS_API EmbeddingImpl : Module {
  using Options = compute::Embedding::Options;
  EmbeddingImpl(const Scheduler &scheduler, const Options &options);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &indices) const;
  void backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const;
  [[nodiscard]] std::shared_ptr<compute::Embedding::State> state() const { return state_.lock(); }

 private:
  std::weak_ptr<compute::Embedding::State> state_;
};
CS_MODULE(Embedding);
}  // namespace cs::module
