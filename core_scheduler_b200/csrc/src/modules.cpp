// SPDX-License-Identifier: Apache-2.0
// Module wrappers. See cs/modules.h.
#include "cs/modules.h"

namespace cs::module {
LinearImpl::LinearImpl(const Scheduler &scheduler, const Options &options) {
  auto state = compute::Linear::init(scheduler, options);
  register_state(state);
  state_ = state;
}
Tensor LinearImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &input) const {
  return compute::Linear::forward(scheduler, state(), input);
}
Tensor LinearImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &input, const ReadOnlyTensor &residual) const {
  return compute::Linear::forward(scheduler, state(), input, residual);
}
Tensor LinearImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  Tensor dx = compute::Linear::backward_input(scheduler, state(), grad_output);
  compute::Linear::backward_parameter(scheduler, state(), grad_output);
  return dx;
}
Tensor LinearImpl::backward_input(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  return compute::Linear::backward_input(scheduler, state(), grad_output);
}
void LinearImpl::backward_parameter(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  compute::Linear::backward_parameter(scheduler, state(), grad_output);
}

GeluLinearImpl::GeluLinearImpl(const Scheduler &scheduler, const Options &options) {
  auto state = compute::GeluLinear::init(scheduler, options);
  register_state(state);
  state_ = state;
}
Tensor GeluLinearImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &input) const {
  return compute::GeluLinear::forward(scheduler, state(), input);
}
Tensor GeluLinearImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &input,
                               const ReadOnlyTensor &residual) const {
  return compute::GeluLinear::forward(scheduler, state(), input, residual);
}
Tensor GeluLinearImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  Tensor dx = compute::GeluLinear::backward_input(scheduler, state(), grad_output);
  compute::GeluLinear::backward_parameter(scheduler, state(), grad_output);
  return dx;
}
Tensor GeluLinearImpl::backward_input(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  return compute::GeluLinear::backward_input(scheduler, state(), grad_output);
}
void GeluLinearImpl::backward_parameter(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  compute::GeluLinear::backward_parameter(scheduler, state(), grad_output);
}

LayerNormImpl::LayerNormImpl(const Scheduler &scheduler, const Options &options) {
  auto state = compute::LayerNorm::init(scheduler, options);
  register_state(state);
  state_ = state;
}
Tensor LayerNormImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &input) const {
  return compute::LayerNorm::forward(scheduler, state(), input);
}
Tensor LayerNormImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  return compute::LayerNorm::backward(scheduler, state(), grad_output);
}
Tensor LayerNormImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output,
                               const ReadOnlyTensor &grad_residual) const {
  return compute::LayerNorm::backward(scheduler, state(), grad_output, grad_residual);
}

EmbeddingImpl::EmbeddingImpl(const Scheduler &scheduler, const Options &options) {
  auto state = compute::Embedding::init(scheduler, options);
  register_state(state);
  state_ = state;
}
Tensor EmbeddingImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &indices) const {
  return compute::Embedding::forward(scheduler, state(), indices);
}
void EmbeddingImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_output) const {
  compute::Embedding::backward(scheduler, state(), grad_output);
}
}  // namespace cs::module
