// SPDX-License-Identifier: Apache-2.0
// Single-device tests of the C++ API against libtorch autograd on the same device (the counterpart of the
// reference project's core_scheduler_tests: test/test_linear.cpp, test_layer_norm.cpp, test_gelu.cpp,
// test_embedding.cpp, test_cross_entropy.cpp, test_flash_attention.cpp, test_utils.cpp, test_autocast.cpp,
// test_adamw.cpp, test_load_save.cpp). The scheduler picks the GPU when there is one and the CPU otherwise;
// 16-bit cases run on GPUs only.
//
//   cs_b200_tests [--filter SUBSTRING]
#include <torch/csrc/distributed/c10d/HashStore.hpp>
#include <torch/torch.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <thread>

#include "cs/compute.h"
#include "cs/data.h"
#include "cs/models.h"
#include "cs/module.h"
#include "cs/modules.h"
#include "cs/optimizer.h"
#include "cs/parallel.h"
#include "cs_test.h"

namespace {
namespace U = cs::compute::Utils;

cs::DynamicScheduler &scheduler() {
  static cs::DynamicScheduler s{0};
  return s;
}
at::Device device() { return scheduler().device(); }
bool on_gpu() { return device().is_cuda(); }
at::TensorOptions opts(at::ScalarType dtype) { return at::TensorOptions{}.dtype(dtype).device(device()); }
at::Tensor host(const cs::ReadOnlyTensor &t) { return cs::memory::to_torch(scheduler(), t); }
cs::Tensor wrap(const at::Tensor &t) { return cs::Tensor::wrap(t.detach().clone()); }
std::vector<at::ScalarType> float_types() { return {at::kFloat, at::kDouble}; }
struct Tolerance {
  double rtol, atol;
};
Tolerance tolerance(at::ScalarType dtype) {
  if (dtype == at::kDouble) return {1e-8, 1e-10};
  if (dtype == at::kFloat) return {1e-4, 1e-5};
  return {2e-2, 2e-2};  // 16-bit
}
}  // namespace

CS_TEST(Linear, MatchesAutogradWithAndWithoutBias) {
  for (auto dtype : float_types())
    for (bool bias : {false, true}) {
      torch::manual_seed(1);
      auto state = cs::compute::Linear::init(scheduler(), cs::compute::Linear::Options{4, 16}.bias(bias).device(device()).dtype(dtype));
      auto x = torch::randn({32, 3, 4}, opts(dtype)).requires_grad_(true);
      auto w = host(state->forward.weight).requires_grad_(true);
      at::Tensor b = bias ? host(state->forward.bias).requires_grad_(true) : at::Tensor{};
      auto reference = torch::linear(x, w, b);
      auto dy = torch::randn_like(reference);
      reference.backward(dy);
      auto y = cs::compute::Linear::forward(scheduler(), state, wrap(x));
      auto dx = cs::compute::Linear::backward_input(scheduler(), state, wrap(dy));
      cs::compute::Linear::backward_parameter(scheduler(), state, wrap(dy));
      const auto tol = tolerance(dtype);
      EXPECT_CLOSE(host(y), reference, tol.rtol, tol.atol);
      EXPECT_CLOSE(host(dx), x.grad(), tol.rtol, tol.atol);
      EXPECT_CLOSE(host(state->forward.grad_weight), w.grad(), tol.rtol, tol.atol);
      if (bias) EXPECT_CLOSE(host(state->forward.grad_bias), b.grad(), tol.rtol, tol.atol);
    }
}

CS_TEST(Linear, WeightGradientAccumulatesOverMicroSteps) {
  auto state = cs::compute::Linear::init(scheduler(), cs::compute::Linear::Options{8, 8}.bias(false).device(device()).dtype(at::kFloat));
  auto x = torch::randn({5, 8}, opts(at::kFloat)), dy = torch::randn({5, 8}, opts(at::kFloat));
  for (int i = 0; i < 2; ++i) {
    cs::compute::Linear::forward(scheduler(), state, wrap(x));
    cs::compute::Linear::backward_parameter(scheduler(), state, wrap(dy));
  }
  EXPECT_CLOSE(host(state->forward.grad_weight), 2 * dy.t().matmul(x), 1e-4, 1e-5);
  state->zero_grad();
  EXPECT_TRUE(!state->forward.grad_weight.defined() || host(state->forward.grad_weight).abs().max().item<double>() == 0.0);
}

CS_TEST(Linear, Bfloat16UnderAutocastKeepsFloat32WeightGradient) {
  if (!on_gpu()) return;  // 16-bit cases need the GPU kernels
  torch::manual_seed(2);
  auto state = cs::compute::Linear::init(scheduler(), cs::compute::Linear::Options{256, 512}.bias(false).device(device()).dtype(at::kFloat));
  auto x = torch::randn({128, 256}, opts(at::kFloat)), dy = torch::randn({128, 512}, opts(at::kFloat));
  cs::Tensor y, dx;
  {
    cs::autocast::ContextGuard guard{scheduler(), at::kBFloat16};
    y = cs::compute::Linear::forward(scheduler(), state, wrap(x.to(at::kBFloat16)));
    dx = cs::compute::Linear::backward_input(scheduler(), state, wrap(dy.to(at::kBFloat16)));
    cs::compute::Linear::backward_parameter(scheduler(), state, wrap(dy.to(at::kBFloat16)));
  }
  const auto w = host(state->forward.weight);
  const auto xb = x.to(at::kBFloat16).to(at::kFloat), dyb = dy.to(at::kBFloat16).to(at::kFloat), wb = w.to(at::kBFloat16).to(at::kFloat);
  EXPECT_TRUE(host(y).scalar_type() == at::kBFloat16);
  EXPECT_CLOSE(host(y).to(at::kFloat), xb.matmul(wb.t()), 2e-2, 2e-1);
  EXPECT_CLOSE(host(dx).to(at::kFloat), dyb.matmul(wb), 2e-2, 2e-1);
  EXPECT_TRUE(host(state->forward.grad_weight).scalar_type() == at::kFloat);
  EXPECT_CLOSE(host(state->forward.grad_weight), dyb.t().matmul(xb), 2e-2, 2e-1);
}

CS_TEST(LayerNorm, MatchesAutograd) {
  for (auto dtype : float_types()) {
    torch::manual_seed(3);
    auto state = cs::compute::LayerNorm::init(scheduler(), cs::compute::LayerNorm::Options{{384}}.device(device()).dtype(dtype));
    U::uniform_(scheduler(), state->forward.weight, 0.5, 1.5);
    U::uniform_(scheduler(), state->forward.bias, -0.5, 0.5);
    auto x = torch::randn({16, 24, 384}, opts(dtype)).requires_grad_(true);
    auto w = host(state->forward.weight).requires_grad_(true), b = host(state->forward.bias).requires_grad_(true);
    auto reference = torch::layer_norm(x, {384}, w, b, 1e-5);
    auto dy = torch::randn_like(reference);
    reference.backward(dy);
    auto y = cs::compute::LayerNorm::forward(scheduler(), state, wrap(x));
    auto dx = cs::compute::LayerNorm::backward(scheduler(), state, wrap(dy));
    const auto tol = tolerance(dtype);
    EXPECT_CLOSE(host(y), reference, tol.rtol, tol.atol * 10);
    EXPECT_CLOSE(host(dx), x.grad(), tol.rtol, tol.atol * 10);
    EXPECT_CLOSE(host(state->forward.grad_weight), w.grad(), tol.rtol, tol.atol * 100);
    EXPECT_CLOSE(host(state->forward.grad_bias), b.grad(), tol.rtol, tol.atol * 100);
  }
}

CS_TEST(GeLU, ForwardAndBackwardMatchAten) {
  for (auto dtype : float_types())
    for (int64_t width : {128, 512, 1024}) {
      auto state = cs::compute::GeLU::init(scheduler());
      auto x = torch::randn({2, width}, opts(dtype)).requires_grad_(true);
      auto reference = at::gelu(x);
      auto dy = torch::randn_like(reference);
      reference.backward(dy);
      auto y = cs::compute::GeLU::forward(scheduler(), state, wrap(x));
      auto dx = cs::compute::GeLU::backward(scheduler(), state, wrap(dy));
      const auto tol = tolerance(dtype);
      EXPECT_CLOSE(host(y), reference, tol.rtol, tol.atol);
      EXPECT_CLOSE(host(dx), x.grad(), tol.rtol, tol.atol);
    }
}

CS_TEST(Embedding, ForwardAndDenseWeightGradient) {
  torch::manual_seed(4);
  auto state = cs::compute::Embedding::init(scheduler(), cs::compute::Embedding::Options{4095, 512}.device(device()).dtype(at::kFloat));
  auto indices = torch::randint(0, 3, {2, 1024}, opts(at::kLong));  // heavy duplication, as in the reference's test
  auto w = host(state->forward.weight).requires_grad_(true);
  auto reference = at::embedding(w, indices);
  auto dy = torch::randn_like(reference);
  reference.backward(dy);
  auto y = cs::compute::Embedding::forward(scheduler(), state, wrap(indices));
  cs::compute::Embedding::backward(scheduler(), state, wrap(dy));
  EXPECT_CLOSE(host(y), reference, 1e-6, 1e-7);
  EXPECT_CLOSE(host(state->forward.grad_weight), w.grad(), 1e-4, 1e-3);
}

CS_TEST(CrossEntropy, LossAndLogitGradient) {
  for (auto dtype : float_types()) {
    torch::manual_seed(5);
    auto state = cs::compute::CrossEntropy::init(scheduler());
    auto logits = torch::randn({2048, 384}, opts(dtype)).requires_grad_(true);
    auto target = torch::randint(0, 384, {2048}, opts(at::kLong));
    auto reference = at::cross_entropy_loss(logits, target);
    reference.backward();
    auto loss = cs::compute::CrossEntropy::forward(scheduler(), state, wrap(logits), wrap(target));
    auto dlogits = cs::compute::CrossEntropy::backward(scheduler(), state);
    const auto tol = tolerance(dtype);
    EXPECT_CLOSE(host(loss), reference, tol.rtol, tol.atol);
    EXPECT_CLOSE(host(dlogits), logits.grad(), tol.rtol, tol.atol);
  }
}

CS_TEST(Attention, CausalMatchesMaskedSoftmaxAutograd) {
  // explicit masked-softmax attention as the oracle (test/test_flash_attention.cpp:61-145 in the reference project)
  const int64_t B = 3, T = 7, H = 4, D = 8;
  const auto dtype = on_gpu() ? at::kBFloat16 : at::kFloat;
  torch::manual_seed(6);
  auto q = torch::randn({B, T, H, D}, opts(dtype)), k = torch::randn({B, T, H, D}, opts(dtype)), v = torch::randn({B, T, H, D}, opts(dtype));
  auto qf = q.to(at::kFloat).requires_grad_(true), kf = k.to(at::kFloat).requires_grad_(true), vf = v.to(at::kFloat).requires_grad_(true);
  auto scores = qf.transpose(1, 2).matmul(kf.transpose(1, 2).transpose(-1, -2)) / std::sqrt(static_cast<double>(D));
  auto mask = torch::ones({T, T}, opts(at::kBool)).tril().logical_not();
  auto reference = scores.masked_fill(mask, -INFINITY).softmax(-1).matmul(vf.transpose(1, 2)).transpose(1, 2);  // [B,T,H,D]
  auto dout = torch::randn({B, T, H, D}, opts(dtype));
  reference.backward(dout.to(at::kFloat));
  auto state = cs::compute::ScaledDotProductAttention::init(scheduler(), cs::compute::ScaledDotProductAttention::Options{}.is_causal(true));
  auto out = cs::compute::ScaledDotProductAttention::forward(scheduler(), state, wrap(q), wrap(k), wrap(v));
  auto grads = cs::compute::ScaledDotProductAttention::backward(scheduler(), state, wrap(dout));
  const double atol = on_gpu() ? 3e-2 : 1e-5, rtol = on_gpu() ? 2e-2 : 1e-4;
  EXPECT_CLOSE(host(out).to(at::kFloat), reference, rtol, atol);
  EXPECT_CLOSE(host(grads[0]).to(at::kFloat), qf.grad(), rtol, atol);
  EXPECT_CLOSE(host(grads[1]).to(at::kFloat), kf.grad(), rtol, atol);
  EXPECT_CLOSE(host(grads[2]).to(at::kFloat), vf.grad(), rtol, atol);
}

CS_TEST(Utils, CatSumAndGradientClipping) {
  for (auto dtype : float_types()) {
    torch::manual_seed(7);
    auto a = torch::randn({32, 16, 8}, opts(dtype)), b = torch::randn({32, 16, 8}, opts(dtype));
    EXPECT_CLOSE(host(U::cat(scheduler(), {wrap(a), wrap(b)}, -1)), at::cat({a, b}, -1), 0, 0);
    EXPECT_CLOSE(host(U::sum(scheduler(), wrap(a), 0)), a.sum(0), tolerance(dtype).rtol, tolerance(dtype).atol * 10);
    // the joint norm over several tensors, then every tensor scaled by max_norm / (norm + 1e-6) when that is below 1
    std::vector<at::Tensor> grads{torch::randn({64, 64}, opts(dtype)), torch::randn({128}, opts(dtype)), torch::randn({3, 5, 7}, opts(dtype))};
    std::vector<cs::Tensor> handles;
    for (auto &g : grads) handles.push_back(wrap(g));
    double squares = 0;
    for (auto &g : grads) squares += g.to(at::kDouble).pow(2).sum().item<double>();
    const double norm = std::sqrt(squares), max_norm = 1.0;
    auto measured = U::clip_grad_norm_(scheduler(), handles, max_norm);
    EXPECT_TRUE(std::abs(host(measured).item<double>() - norm) < 1e-4 * norm);
    const double coefficient = std::min(1.0, max_norm / (norm + 1e-6));
    for (size_t i = 0; i < grads.size(); ++i) EXPECT_CLOSE(host(handles[i]), grads[i] * coefficient, 1e-4, 1e-6);
  }
}

CS_TEST(Utils, FactoriesViewsAndSplit) {
  auto r = U::arange(scheduler(), 0, 24, opts(at::kFloat));
  EXPECT_CLOSE(host(r), torch::arange(0, 24, opts(at::kFloat)), 0, 0);
  auto v = U::view(scheduler(), r, {2, 3, 4});
  EXPECT_TRUE(host(v).sizes() == at::IntArrayRef({2, 3, 4}));
  auto parts = U::split(scheduler(), v, 2, -1);
  EXPECT_TRUE(parts.size() == 2);
  EXPECT_CLOSE(host(parts[1]), torch::arange(0, 24, opts(at::kFloat)).view({2, 3, 4}).split(2, -1)[1], 0, 0);
  EXPECT_CLOSE(host(U::add(scheduler(), U::ones(scheduler(), {4}, opts(at::kFloat)), U::zeros(scheduler(), {4}, opts(at::kFloat)))),
               torch::ones({4}, opts(at::kFloat)), 0, 0);
  EXPECT_CLOSE(host(U::broadcast_to(scheduler(), U::ones(scheduler(), {1, 4}, opts(at::kFloat)), {3, 4})), torch::ones({3, 4}), 0, 0);
  auto ids = host(U::randint(scheduler(), 5, 9, {1000}, opts(at::kLong)));
  EXPECT_TRUE(ids.min().item<int64_t>() >= 5 && ids.max().item<int64_t>() < 9);
}

CS_TEST(Autocast, GuardSetsAndRestoresTheSchedulersState) {
  // the autocast state belongs to the scheduler (ops read it when their task is submitted), not to the ATen thread
  EXPECT_TRUE(!scheduler().impl()->autocast_enabled);
  {
    cs::autocast::ContextGuard guard{scheduler(), at::kBFloat16};
    EXPECT_TRUE(scheduler().impl()->autocast_enabled && scheduler().impl()->autocast_dtype == at::kBFloat16);
    {
      cs::autocast::ContextGuard inner{scheduler(), at::kHalf};
      EXPECT_TRUE(scheduler().impl()->autocast_dtype == at::kHalf);
    }
    EXPECT_TRUE(scheduler().impl()->autocast_enabled && scheduler().impl()->autocast_dtype == at::kBFloat16);
    if (on_gpu()) {  // fp32 parameters, 16-bit activations: statistics in fp32, output in the activation type
      auto norm = cs::compute::LayerNorm::init(scheduler(), cs::compute::LayerNorm::Options{{256}}.device(device()).dtype(at::kFloat));
      auto x = torch::randn({64, 256}, opts(at::kBFloat16));
      auto y = cs::compute::LayerNorm::forward(scheduler(), norm, wrap(x));
      auto reference = torch::layer_norm(x.to(at::kFloat), {256}, host(norm->forward.weight), host(norm->forward.bias), 1e-5);
      EXPECT_CLOSE(host(y).to(at::kFloat), reference, 2e-2, 2e-2);
    }
  }
  EXPECT_TRUE(!scheduler().impl()->autocast_enabled);
}

CS_TEST(AdamW, FunctionalStepMatchesTheFormula) {
  for (bool amsgrad : {false, true})
    for (int64_t n : {128, 512, 1024}) {
      torch::manual_seed(8);
      const double lr = 1e-2, beta1 = 0.9, beta2 = 0.95, eps = 1e-8, wd = 0.1;
      auto w0 = torch::randn({n}, opts(at::kFloat));
      auto w = wrap(w0);
      auto state = cs::optimizer::AdamW::init(
          scheduler(), w, cs::optimizer::AdamW::Options{}.lr(lr).beta1(beta1).beta2(beta2).eps(eps).weight_decay(wd).amsgrad(amsgrad));
      auto ref_w = w0.to(at::kDouble).cpu(), m = torch::zeros({n}, at::kDouble), v = torch::zeros({n}, at::kDouble), v_max = torch::zeros({n}, at::kDouble);
      for (int t = 1; t <= 3; ++t) {
        auto g = torch::randn({n}, opts(at::kFloat));
        cs::optimizer::AdamW::step(scheduler(), state, w, wrap(g));
        auto gd = g.to(at::kDouble).cpu();
        ref_w = ref_w - lr * wd * ref_w;
        m = beta1 * m + (1 - beta1) * gd;
        v = beta2 * v + (1 - beta2) * gd * gd;
        auto m_hat = m / (1 - std::pow(beta1, t)), v_hat = v / (1 - std::pow(beta2, t));
        if (amsgrad) {
          v_max = at::maximum(v_max, v_hat);
          v_hat = v_max;
        }
        ref_w = ref_w - lr * m_hat / (v_hat.sqrt() + eps);
      }
      EXPECT_CLOSE(host(w), ref_w, 1e-4, 1e-5);
      EXPECT_CLOSE(host(state->tensors.m), m, 1e-4, 1e-6);
      EXPECT_CLOSE(host(state->tensors.v), v, 1e-4, 1e-7);
    }
}

CS_TEST(AdamW, ModuleStepMatchesTorchOptim) {
  torch::manual_seed(9);
  cs::module::Linear layer{scheduler(), cs::compute::Linear::Options{64, 32}.bias(true).device(device()).dtype(at::kFloat)};
  cs::module::AdamW optimizer{scheduler(), layer, cs::optimizer::AdamW::Options{}.lr(1e-2).beta1(0.9).beta2(0.95).weight_decay(0.1)};
  auto w = host(layer->state()->forward.weight).requires_grad_(true), b = host(layer->state()->forward.bias).requires_grad_(true);
  torch::optim::AdamW reference{{w, b}, torch::optim::AdamWOptions(1e-2).betas({0.9, 0.95}).weight_decay(0.1).eps(1e-8)};
  for (int step = 0; step < 3; ++step) {
    auto x = torch::randn({16, 64}, opts(at::kFloat)), dy = torch::randn({16, 32}, opts(at::kFloat));
    reference.zero_grad();
    torch::linear(x, w, b).backward(dy);
    reference.step();
    layer->forward(scheduler(), wrap(x));
    layer->backward(scheduler(), wrap(dy));
    optimizer->step(scheduler());
    optimizer->zero_grad(scheduler());
  }
  EXPECT_CLOSE(host(layer->state()->forward.weight), w, 1e-4, 1e-5);
  EXPECT_CLOSE(host(layer->state()->forward.bias), b, 1e-4, 1e-5);
}

CS_TEST(Checkpoint, SaveZeroLoadRestoresTheParameters) {
  for (auto dtype : float_types()) {
    cs::module::LayerNorm layer{scheduler(), cs::compute::LayerNorm::Options{{384}}.device(device()).dtype(dtype)};
    U::uniform_(scheduler(), layer->state()->forward.weight, 0.5, 1.5);
    U::normal_(scheduler(), layer->state()->forward.bias, 0.0, 1.0);
    const auto weight = host(layer->state()->forward.weight), bias = host(layer->state()->forward.bias);
    const std::string path = "/tmp/cs_b200_tests_" + std::to_string(::getpid()) + "_model.parquet";
    cs::save(layer, path);
    U::zero_(scheduler(), layer->state()->forward.weight);
    U::zero_(scheduler(), layer->state()->forward.bias);
    EXPECT_TRUE(host(layer->state()->forward.weight).abs().max().item<double>() == 0.0);
    cs::load(layer, path);
    std::remove(path.c_str());
    // the file stores float32 values, as the reference's does
    EXPECT_CLOSE(host(layer->state()->forward.weight), weight, 1e-6, 1e-7);
    EXPECT_CLOSE(host(layer->state()->forward.bias), bias, 1e-6, 1e-7);
    EXPECT_TRUE(host(layer->state()->forward.weight).scalar_type() == dtype);
  }
}

CS_TEST(Scheduler, AssistStreamResultsReachTheMainStreamInOrder) {
  // a chain that alternates between the assist stream (weight gradients) and the main stream (their consumers)
  auto state = cs::compute::Linear::init(scheduler(), cs::compute::Linear::Options{32, 32}.bias(false).device(device()).dtype(at::kFloat));
  auto x = torch::randn({64, 32}, opts(at::kFloat)), dy = torch::randn({64, 32}, opts(at::kFloat));
  at::Tensor expected = torch::zeros({32, 32}, opts(at::kFloat));
  for (int i = 0; i < 20; ++i) {
    cs::compute::Linear::forward(scheduler(), state, wrap(x));
    cs::compute::Linear::backward_parameter(scheduler(), state, wrap(dy));                                     // assist stream
    auto doubled = U::add(scheduler(), state->forward.grad_weight, state->forward.grad_weight);            // main stream reads it
    expected = expected + dy.t().matmul(x);
    EXPECT_CLOSE(host(doubled), 2 * expected, 1e-4, 1e-3);
  }
}

CS_TEST(GeluLinear, MatchesLinearOfGeluAutograd) {
  for (bool bias : {false, true}) {
    torch::manual_seed(10);
    const auto dtype = at::kDouble;
    auto state = cs::compute::GeluLinear::init(scheduler(), cs::compute::GeluLinear::Options{128, 64}.bias(bias).device(device()).dtype(dtype));
    auto x = torch::randn({12, 3, 128}, opts(dtype)).requires_grad_(true);
    auto w = host(state->forward.weight).requires_grad_(true);
    at::Tensor b = bias ? host(state->forward.bias).requires_grad_(true) : at::Tensor{};
    auto reference = torch::linear(at::gelu(x), w, b);
    auto dy = torch::randn_like(reference);
    reference.backward(dy);
    auto y = cs::compute::GeluLinear::forward(scheduler(), state, wrap(x));
    auto dx = cs::compute::GeluLinear::backward_input(scheduler(), state, wrap(dy));
    cs::compute::GeluLinear::backward_parameter(scheduler(), state, wrap(dy));
    EXPECT_CLOSE(host(y), reference, 1e-8, 1e-10);
    EXPECT_CLOSE(host(dx), x.grad(), 1e-8, 1e-10);
    EXPECT_CLOSE(host(state->forward.grad_weight), w.grad(), 1e-8, 1e-10);
    if (bias) EXPECT_CLOSE(host(state->forward.grad_bias), b.grad(), 1e-8, 1e-10);
  }
}

CS_TEST(Module, ParameterKeysAreDottedPathsInRegistrationOrder) {
  struct Block : cs::module::Module {
    cs::module::LayerNorm norm{nullptr};
    cs::module::Linear proj{nullptr};
    explicit Block(const cs::Scheduler &s) {
      norm = register_module("ln", cs::module::LayerNorm{s, cs::compute::LayerNorm::Options{{8}}.device(device()).dtype(at::kFloat)});
      proj = register_module("c_proj", cs::module::Linear{s, cs::compute::Linear::Options{8, 8}.bias(false).device(device()).dtype(at::kFloat)});
    }
  };
  struct Net : cs::module::Module {
    explicit Net(const cs::Scheduler &s) {
      register_module("wte", cs::module::Embedding{s, cs::compute::Embedding::Options{16, 8}.device(device()).dtype(at::kFloat)});
      for (int i = 0; i < 2; ++i) register_module(std::to_string(i), std::make_shared<Block>(s));
    }
  };
  auto net = std::make_shared<Net>(scheduler());
  std::vector<std::string> keys;
  for (auto &item : net->named_parameters()) keys.push_back(item.key());
  const std::vector<std::string> expected{"wte.weight", "0.ln.weight", "0.ln.bias", "0.c_proj.weight", "1.ln.weight", "1.ln.bias", "1.c_proj.weight"};
  EXPECT_TRUE(keys == expected);
}

CS_TEST(DataLoader, ProducerThreadHandsOverBatchesThroughTheTwoSlots) {
  // the worker thread fills one slot while load() uploads the other; labels are the inputs shifted by one token,
  // two loaders with one seed deliver the same stream, and a loader that is destroyed mid-stream joins its worker
  const int64_t batch = 3, seq = 17, vocab = 97;
  cs::data::SyntheticDataLoader a{batch, seq, vocab, 5}, b{batch, seq, vocab, 5};
  for (int i = 0; i < 12; ++i) {
    auto xa = a.load(scheduler()), xb = b.load(scheduler());
    at::Tensor ids = host(xa.at("input_ids")).cpu(), labels = host(xa.at("labels")).cpu();
    EXPECT_TRUE(ids.sizes() == at::IntArrayRef({batch, seq}) && labels.sizes() == ids.sizes());
    EXPECT_TRUE(ids.min().item<int64_t>() >= 0 && ids.max().item<int64_t>() < vocab);
    EXPECT_TRUE(at::equal(ids.slice(1, 1, seq), labels.slice(1, 0, seq - 1)));
    EXPECT_TRUE(at::equal(ids, host(xb.at("input_ids")).cpu()));
  }
  {
    cs::data::SyntheticDataLoader c{batch, seq, vocab, 6};
    (void)c.load(scheduler());
  }
}

CS_TEST(Parallel, RanksAgreeOnTheLargestAllocationSize) {
  // symmetric arenas stay aligned across ranks only if every rank allocates the same sizes: shards of different
  // sizes (20 heads over 8 ranks) are allocated with the largest size any rank asked for
  auto store = c10::make_intrusive<c10d::HashStore>();
  std::vector<int64_t> got(3, 0);
  std::vector<std::thread> ranks;
  for (int r = 0; r < 3; ++r)
    ranks.emplace_back([&, r] { got[r] = cs::parallel::agree_on_max(store.get(), "arena/0/", r, 3, 1000 + 64 * (r % 2)); });
  for (auto &t : ranks) t.join();
  for (int r = 0; r < 3; ++r) EXPECT_TRUE(got[r] == 1064);
  EXPECT_TRUE(cs::parallel::agree_on_max(nullptr, "arena/1/", 0, 4, 7) == 7);      // no store: nothing to agree with
  EXPECT_TRUE(cs::parallel::agree_on_max(store.get(), "arena/2/", 0, 1, 9) == 9);  // one rank
}

CS_TEST(Model, TinyGpt2LossFallsOverAFewSteps) {
  cs::manual_seed(11);
  cs::models::GPT2 model{scheduler(), cs::models::GPT2Config::tiny()};
  auto flat = cs::module::flatten_parameters(scheduler(), *model, cs::module::FlattenOptions{});
  cs::module::AdamW optimizer{scheduler(), *model, flat, cs::optimizer::AdamW::Options{}.lr(3e-3).beta1(0.9).beta2(0.95).weight_decay(0.0)};
  cs::data::SyntheticDataLoader loader{4, 64, 512, 5};
  auto batch = loader.load(scheduler());  // one fixed batch: the model has to memorise it
  double first = 0, last = 0;
  for (int step = 0; step < 8; ++step) {
    auto loss = model->forward_loss(scheduler(), batch["input_ids"], batch["labels"]);
    model->backward_loss(scheduler());
    optimizer->step(scheduler());
    optimizer->zero_grad(scheduler());
    last = host(loss).item<double>();
    if (step == 0) first = last;
  }
  EXPECT_TRUE(std::abs(first - std::log(512.0)) < 0.3);  // random init: close to log(vocab)
  EXPECT_TRUE(last < first - 0.5);
}

int main(int argc, char **argv) {
  std::printf("device: %s\n", device().str().c_str());
  return cs_test::run_all(argc, argv);
}
