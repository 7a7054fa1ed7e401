// SPDX-License-Identifier: Apache-2.0
// GPT-2 model. See cs/models.h for the parity map and the fusion list.
#include <cmath>

#include "cs/models.h"

namespace cs::models {
namespace Utils = compute::Utils;

GPT2Config GPT2Config::tiny() {
  return GPT2Config{}.n_layer(2).n_head(4).n_embd(128).block_size(64).vocab_size(512).padded_vocab_size(512);
}
GPT2Config GPT2Config::gpt2_124m() { return GPT2Config{}; }
GPT2Config GPT2Config::gpt2_350m() { return GPT2Config{}.n_layer(24).n_head(16).n_embd(1024); }
GPT2Config GPT2Config::gpt2_774m() { return GPT2Config{}.n_layer(36).n_head(20).n_embd(1280); }

int64_t GPT2Config::parameter_count() const {
  const int64_t d = n_embd_;
  int64_t per_block = 4 * d /*ln1, ln2*/ + 3 * d * d + d * d + 4 * d * d + 4 * d * d;
  if (use_bias_) per_block += 3 * d + d + 4 * d + d;
  return padded_vocab_size_ * d /*wte*/ + block_size_ * d /*wpe*/ + n_layer_ * per_block + 2 * d /*lnf*/ +
         padded_vocab_size_ * d /*lm_head*/;
}

double GPT2Config::train_flops_per_token(int64_t seq_len) const {
  const double d = static_cast<double>(n_embd_);
  const double matmul_params = static_cast<double>(n_layer_) * 12.0 * d * d + static_cast<double>(padded_vocab_size_) * d;
  const double attention = 4.0 * static_cast<double>(n_layer_) * static_cast<double>(seq_len) * d;
  return 3.0 * (2.0 * matmul_params + attention);
}

namespace {
at::Device device_of(const Scheduler &scheduler, const GPT2Config &c) { return c.device().value_or(scheduler.device()); }

compute::Linear::Options linear_options(const Scheduler &scheduler, const GPT2Config &c, int64_t in, int64_t out) {
  return compute::Linear::Options{in, out}.bias(c.use_bias()).device(device_of(scheduler, c)).dtype(c.dtype());
}
}  // namespace

// ----------------------------------------------------------------------------- attention ----
AttnImpl::AttnImpl(const Scheduler &scheduler, const GPT2Config &config) : n_head{config.n_head()} {
  const int64_t d = config.n_embd();
  CS_ASSERT_TRUE(d % n_head == 0, "n_embd must be divisible by n_head");
  c_attn = register_module("c_attn", module::Linear{scheduler, linear_options(scheduler, config, d, 3 * d)});
  c_proj = register_module("c_proj", module::Linear{scheduler, linear_options(scheduler, config, d, d)});
  attn_state = compute::ScaledDotProductAttention::init(
      scheduler, compute::ScaledDotProductAttention::Options{}.is_causal(true));
  const double std = config.scale_residual_init() ? config.init_std() / std::sqrt(2.0 * config.n_layer())
                                                  : config.init_std();
  Utils::normal_(scheduler, c_attn->state()->forward.weight, 0, config.init_std());
  Utils::normal_(scheduler, c_proj->state()->forward.weight, 0, std);
  if (config.use_bias()) {
    Utils::zero_(scheduler, c_attn->state()->forward.bias);
    Utils::zero_(scheduler, c_proj->state()->forward.bias);
  }
}

Tensor AttnImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &x, const ReadOnlyTensor &residual) {
  Tensor qkv = c_attn->forward(scheduler, x);  // [B,T,3d]
  Tensor ctx = compute::ScaledDotProductAttention::forward_packed(scheduler, attn_state, qkv, n_head);  // [B,T,d]
  return c_proj->forward(scheduler, ctx, residual);  // residual add fused into the epilogue
}

Tensor AttnImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad, const GradientSync &sync) {
  Tensor d_ctx = c_proj->backward_input(scheduler, grad);
  c_proj->backward_parameter(scheduler, grad);
  sync.push(scheduler, c_proj->state()->forward.grad_weight);
  if (c_proj->state()->args.bias) sync.push(scheduler, c_proj->state()->forward.grad_bias);
  Tensor d_qkv = compute::ScaledDotProductAttention::backward_packed(scheduler, attn_state, d_ctx);
  Tensor d_x = c_attn->backward_input(scheduler, d_qkv);
  c_attn->backward_parameter(scheduler, d_qkv);
  sync.push(scheduler, c_attn->state()->forward.grad_weight);
  if (c_attn->state()->args.bias) sync.push(scheduler, c_attn->state()->forward.grad_bias);
  return d_x;
}

// ----------------------------------------------------------------------------------- MLP ----
MLPImpl::MLPImpl(const Scheduler &scheduler, const GPT2Config &config) {
  const int64_t d = config.n_embd();
  fc1 = register_module("fc1", module::Linear{scheduler, linear_options(scheduler, config, d, 4 * d).gelu_epilogue(true)});
  fc2 = register_module("fc2", module::GeluLinear{scheduler, linear_options(scheduler, config, 4 * d, d)});
  const double std = config.scale_residual_init() ? config.init_std() / std::sqrt(2.0 * config.n_layer())
                                                  : config.init_std();
  Utils::normal_(scheduler, fc1->state()->forward.weight, 0, config.init_std());
  Utils::normal_(scheduler, fc2->state()->forward.weight, 0, std);
  if (config.use_bias()) {
    Utils::zero_(scheduler, fc1->state()->forward.bias);
    Utils::zero_(scheduler, fc2->state()->forward.bias);
  }
}

Tensor MLPImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &x, const ReadOnlyTensor &residual) {
  Tensor pre = fc1->forward(scheduler, x);          // carries GELU(pre) as companion
  return fc2->forward(scheduler, pre, residual);    // GELU(pre) W2^T + residual
}

Tensor MLPImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad, const GradientSync &sync) {
  Tensor d_pre = fc2->backward_input(scheduler, grad);  // includes GELU'
  fc2->backward_parameter(scheduler, grad);
  sync.push(scheduler, fc2->state()->forward.grad_weight);
  if (fc2->state()->args.bias) sync.push(scheduler, fc2->state()->forward.grad_bias);
  Tensor d_x = fc1->backward_input(scheduler, d_pre);
  fc1->backward_parameter(scheduler, d_pre);
  sync.push(scheduler, fc1->state()->forward.grad_weight);
  if (fc1->state()->args.bias) sync.push(scheduler, fc1->state()->forward.grad_bias);
  return d_x;
}

// --------------------------------------------------------------------------------- block ----
BlockImpl::BlockImpl(const Scheduler &scheduler, const GPT2Config &config) {
  auto ln_opts = compute::LayerNorm::Options{config.n_embd()}.device(device_of(scheduler, config)).dtype(config.dtype());
  ln1 = register_module("ln1", module::LayerNorm{scheduler, ln_opts});
  attn = register_module("attn", Attn{scheduler, config});
  ln2 = register_module("ln2", module::LayerNorm{scheduler, ln_opts});
  mlp = register_module("mlp", MLP{scheduler, config});
}

Tensor BlockImpl::forward(const Scheduler &scheduler, const ReadOnlyTensor &x) {
  Tensor a = ln1->forward(scheduler, x);
  Tensor x1 = attn->forward(scheduler, a, x);   // x + attn(ln1(x))
  Tensor b = ln2->forward(scheduler, x1);
  return mlp->forward(scheduler, b, x1);        // x1 + mlp(ln2(x1))
}

Tensor BlockImpl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad, const GradientSync &sync) {
  Tensor d_b = mlp->backward(scheduler, grad, sync);
  Tensor d_x1 = ln2->backward(scheduler, d_b, grad);  // + residual branch
  sync.push(scheduler, ln2->state()->forward.grad_weight);
  sync.push(scheduler, ln2->state()->forward.grad_bias);
  Tensor d_a = attn->backward(scheduler, d_x1, sync);
  Tensor d_x = ln1->backward(scheduler, d_a, d_x1);
  sync.push(scheduler, ln1->state()->forward.grad_weight);
  sync.push(scheduler, ln1->state()->forward.grad_bias);
  return d_x;
}

// --------------------------------------------------------------------------------- model ----
GPT2Impl::GPT2Impl(const Scheduler &scheduler, const GPT2Config &config) : config_{config} {
  const auto dev = device_of(scheduler, config);
  const int64_t d = config.n_embd();
  wte = register_module("wte", module::Embedding{scheduler, compute::Embedding::Options{config.padded_vocab_size(), d}
                                                                .device(dev)
                                                                .dtype(config.dtype())});
  wpe = register_module("wpe", module::Embedding{scheduler, compute::Embedding::Options{config.block_size(), d}
                                                                .device(dev)
                                                                .dtype(config.dtype())});
  Utils::normal_(scheduler, wte->state()->forward.weight, 0, config.init_std());
  Utils::normal_(scheduler, wpe->state()->forward.weight, 0, config.init_std());
  for (int64_t layer = 0; layer < config.n_layer(); ++layer) {
    h.push_back(register_module(std::to_string(layer), Block{scheduler, config}));
  }
  lnf = register_module("lnf", module::LayerNorm{scheduler, compute::LayerNorm::Options{d}.device(dev).dtype(config.dtype())});
  lm_head = register_module(
      "lm_head", module::Linear{scheduler, compute::Linear::Options{d, config.padded_vocab_size()}.bias(false).device(dev).dtype(
                                               config.dtype())});
  Utils::normal_(scheduler, lm_head->state()->forward.weight, 0, config.init_std());
  lce_state_ = compute::LinearCrossEntropy::init(scheduler, lm_head->state(), config.vocab_size(), -100);
  ce_state_ = compute::CrossEntropy::init(scheduler);
  positions_ = Utils::arange(scheduler, 0, config.block_size(), at::TensorOptions().dtype(at::kLong).device(dev));
}

Tensor GPT2Impl::embed(const Scheduler &scheduler, const ReadOnlyTensor &input_ids) {
  CS_ASSERT_TRUE(input_ids.defined() && input_ids.sizes().size() == 2, "input_ids must be a materialised [B,T] tensor");
  const int64_t T = input_ids.size(1);
  CS_ASSERT_TRUE(T <= config_.block_size(), "sequence length ", T, " exceeds block_size ", config_.block_size());
  fused_embedding_ = true;
  last_batch_ = input_ids.size(0);
  last_seq_ = T;
  return compute::Embedding::forward_token_position(scheduler, wte->state(), wpe->state(), input_ids);
}

Tensor GPT2Impl::forward(const Scheduler &scheduler, const ReadOnlyTensor &input_ids) {
  Tensor x = embed(scheduler, input_ids);
  for (auto &block : h) x = block->forward(scheduler, x);
  x = lnf->forward(scheduler, x);
  return lm_head->forward(scheduler, x);
}

void GPT2Impl::backward_trunk(const Scheduler &scheduler, Tensor grad, const GradientSync &sync) {
  grad = lnf->backward(scheduler, grad);
  sync.push(scheduler, lnf->state()->forward.grad_weight);
  sync.push(scheduler, lnf->state()->forward.grad_bias);
  for (auto it = h.rbegin(); it != h.rend(); ++it) grad = (*it)->backward(scheduler, grad, sync);
  compute::Embedding::backward_token_position(scheduler, wte->state(), wpe->state(), grad);
  sync.push(scheduler, wpe->state()->forward.grad_weight);
  sync.push(scheduler, wte->state()->forward.grad_weight);
}

void GPT2Impl::backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_logits, const GradientSync &sync) {
  Tensor grad = lm_head->backward_input(scheduler, grad_logits);
  lm_head->backward_parameter(scheduler, grad_logits);
  sync.push(scheduler, lm_head->state()->forward.grad_weight);
  grad = Utils::view(scheduler, grad, {last_batch_, last_seq_, config_.n_embd()});
  backward_trunk(scheduler, grad, sync);
}

Tensor GPT2Impl::forward_loss(const Scheduler &scheduler, const ReadOnlyTensor &input_ids, const ReadOnlyTensor &labels) {
  Tensor x = embed(scheduler, input_ids);
  for (auto &block : h) x = block->forward(scheduler, x);
  x = lnf->forward(scheduler, x);
  if (config_.fused_classifier()) return compute::LinearCrossEntropy::forward(scheduler, lce_state_, x, labels);
  Tensor logits = lm_head->forward(scheduler, x);
  const int64_t rows = input_ids.numel();
  Tensor flat = Utils::view(scheduler, logits, {rows, config_.padded_vocab_size()});
  Tensor target = Utils::view(scheduler, labels, {rows});
  return compute::CrossEntropy::forward(scheduler, ce_state_, flat, target);
}

void GPT2Impl::backward_loss(const Scheduler &scheduler, const GradientSync &sync) {
  if (config_.fused_classifier()) {
    Tensor grad = compute::LinearCrossEntropy::backward(scheduler, lce_state_);
    sync.push(scheduler, lm_head->state()->forward.grad_weight);
    backward_trunk(scheduler, grad, sync);
    return;
  }
  Tensor d_logits = compute::CrossEntropy::backward(scheduler, ce_state_);
  backward(scheduler, d_logits, sync);
}
}  // namespace cs::models
