// SPDX-License-Identifier: Apache-2.0
// Pure-libtorch autograd GPT-2 for comparison (counterpart of the reference project's
// example/gpt2/baseline.cpp): bf16 parameters, torch::optim::AdamW, synthetic random tokens,
// the same tokens/sec print as the framework examples. Nothing of this library's runtime is
// used except the configuration struct.
#include <torch/torch.h>

#include <chrono>
#include <iostream>

#include "cs/models.h"

struct Block : torch::nn::Module {
  Block(int64_t d, int64_t heads) : heads{heads} {
    ln1 = register_module("ln1", torch::nn::LayerNorm(torch::nn::LayerNormOptions({d})));
    ln2 = register_module("ln2", torch::nn::LayerNorm(torch::nn::LayerNormOptions({d})));
    c_attn = register_module("c_attn", torch::nn::Linear(torch::nn::LinearOptions(d, 3 * d).bias(false)));
    c_proj = register_module("c_proj", torch::nn::Linear(torch::nn::LinearOptions(d, d).bias(false)));
    fc1 = register_module("fc1", torch::nn::Linear(torch::nn::LinearOptions(d, 4 * d).bias(false)));
    fc2 = register_module("fc2", torch::nn::Linear(torch::nn::LinearOptions(4 * d, d).bias(false)));
  }
  torch::Tensor forward(const torch::Tensor &x) {
    const auto B = x.size(0), T = x.size(1), d = x.size(2);
    auto qkv = c_attn->forward(ln1->forward(x)).view({B, T, 3, heads, d / heads}).permute({2, 0, 3, 1, 4});
    auto ctx = at::scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], {}, 0.0, true);
    auto h = x + c_proj->forward(ctx.transpose(1, 2).reshape({B, T, d}));
    return h + fc2->forward(torch::gelu(fc1->forward(ln2->forward(h))));
  }
  int64_t heads;
  torch::nn::LayerNorm ln1{nullptr}, ln2{nullptr};
  torch::nn::Linear c_attn{nullptr}, c_proj{nullptr}, fc1{nullptr}, fc2{nullptr};
};

struct Net : torch::nn::Module {
  explicit Net(const cs::models::GPT2Config &c) {
    wte = register_module("wte", torch::nn::Embedding(c.padded_vocab_size(), c.n_embd()));
    wpe = register_module("wpe", torch::nn::Embedding(c.block_size(), c.n_embd()));
    for (int64_t l = 0; l < c.n_layer(); ++l)
      blocks.push_back(register_module(std::to_string(l), std::make_shared<Block>(c.n_embd(), c.n_head())));
    lnf = register_module("lnf", torch::nn::LayerNorm(torch::nn::LayerNormOptions({c.n_embd()})));
    lm_head = register_module("lm_head", torch::nn::Linear(torch::nn::LinearOptions(c.n_embd(), c.padded_vocab_size()).bias(false)));
  }
  torch::Tensor forward(const torch::Tensor &ids) {
    auto pos = torch::arange(ids.size(1), ids.options());
    auto x = wte->forward(ids) + wpe->forward(pos);
    for (auto &b : blocks) x = b->forward(x);
    return lm_head->forward(lnf->forward(x));
  }
  torch::nn::Embedding wte{nullptr}, wpe{nullptr};
  std::vector<std::shared_ptr<Block>> blocks;
  torch::nn::LayerNorm lnf{nullptr};
  torch::nn::Linear lm_head{nullptr};
};

int main(int argc, char **argv) {
  int64_t steps = argc > 1 ? std::atoll(argv[1]) : 10, batch = argc > 2 ? std::atoll(argv[2]) : 8;
  const bool cuda = torch::cuda::is_available();
  auto config = cuda ? cs::models::GPT2Config::gpt2_124m() : cs::models::GPT2Config::tiny();
  const auto device = cuda ? torch::kCUDA : torch::kCPU;
  Net net{config};
  net.to(device, cuda ? torch::kBFloat16 : torch::kFloat32);
  torch::optim::AdamW opt(net.parameters(), torch::optim::AdamWOptions(3e-4).betas({0.9, 0.95}).weight_decay(0.1));
  const int64_t T = config.block_size();
  for (int64_t step = 0; step < steps; ++step) {
    const auto t0 = std::chrono::steady_clock::now();
    auto ids = torch::randint(0, config.vocab_size(), {batch, T + 1}, torch::TensorOptions().dtype(torch::kLong).device(device));
    auto logits = net.forward(ids.narrow(1, 0, T));
    auto loss = torch::nn::functional::cross_entropy(logits.reshape({batch * T, -1}).to(torch::kFloat32), ids.narrow(1, 1, T).reshape({-1}));
    opt.zero_grad();
    loss.backward();
    opt.step();
    const double value = loss.item<double>();
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::printf("step %4ld/%ld | loss %.6f | %.2f ms | %.0f tok/s\n", static_cast<long>(step + 1), static_cast<long>(steps), value,
                dt * 1e3, static_cast<double>(batch * T) / dt);
  }
  return 0;
}
