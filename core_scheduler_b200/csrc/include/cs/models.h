// SPDX-License-Identifier: Apache-2.0
// GPT-2 built from this library's modules with a hand-written backward pass (no autograd).
//
// Structure, parameter names and backward order follow the reference project's example
// (example/gpt2/gpt2_single_device.cpp:272-576, example/gpt2/gpt2_ddp.cpp:271-592): wte, wpe,
// blocks named by their index with ln1 / attn{c_attn,c_proj} / ln2 / mlp{fc1,fc2}, lnf, an
// untied lm_head, no Linear biases, LayerNorm with bias. For every Linear the input gradient is
// issued on the main stream before the weight gradient on the assist stream, and on the last
// micro-step each gradient is queued for the bucketed all-reduce right after it is produced.
// Blocks are walked in reverse order in backward (the reference's DDP example walks them
// forward, which is wrong).
//
// Fusions used when tensors are bf16 on a GPU: token+position embedding in one kernel; residual
// adds inside the c_proj / fc2 GEMM epilogues; GELU emitted by the fc1 epilogue; attention on
// the packed qkv tensor; LayerNorm backward with the residual-branch add; classifier GEMM fused
// with the cross-entropy.
#pragma once
#include "cs/communication.h"
#include "cs/compute.h"
#include "cs/modules.h"
#include "cs/optimizer.h"

namespace cs::models {
struct GPT2Config {
  GPT2Config() {}
  CS_ARG(int64_t, n_layer) = 12;
  CS_ARG(int64_t, n_head) = 12;
  CS_ARG(int64_t, n_embd) = 768;
  CS_ARG(int64_t, block_size) = 1024;
  CS_ARG(int64_t, vocab_size) = 50257;         // real vocabulary
  CS_ARG(int64_t, padded_vocab_size) = 50304;  // classifier/embedding rows
  CS_ARG(bool, use_bias) = false;
  CS_ARG(at::ScalarType, dtype) = at::kFloat;  // parameter dtype
  CS_ARG(optional<at::Device>, device) = {};
  CS_ARG(double, init_std) = 0.02;
  CS_ARG(bool, scale_residual_init) = false;   // c_proj/fc2 ~ N(0, std/sqrt(2 n_layer))
  CS_ARG(bool, fused_classifier) = true;

 public:
  static GPT2Config tiny();      // 2 layers, d=128, 4 heads, vocab 512, seq 64
  static GPT2Config gpt2_124m();
  static GPT2Config gpt2_350m();
  static GPT2Config gpt2_774m();
  [[nodiscard]] int64_t parameter_count() const;
  // forward+backward matmul and attention FLOPs per token (causal attention counted in full)
  [[nodiscard]] double train_flops_per_token(int64_t seq_len) const;
};

// What backward needs to overlap gradient communication with compute.
struct GradientSync {
  communication::Comm comm;
  const communication::AllReduceBucket *bucket{nullptr};
  bool last_micro_step{true};
  void push(const Scheduler &scheduler, const Tensor &grad) const {
    if (bucket && last_micro_step && comm.defined()) bucket->push_back(scheduler, comm, grad);
  }
};

struct CS_API AttnImpl : module::Module {
  AttnImpl(const Scheduler &scheduler, const GPT2Config &config);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &x, const ReadOnlyTensor &residual);
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad, const GradientSync &sync);
  module::Linear c_attn{nullptr}, c_proj{nullptr};
  std::shared_ptr<compute::ScaledDotProductAttention::State> attn_state;
  int64_t n_head;
};
CS_MODULE(Attn);

struct CS_API MLPImpl : module::Module {
  MLPImpl(const Scheduler &scheduler, const GPT2Config &config);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &x, const ReadOnlyTensor &residual);
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad, const GradientSync &sync);
  module::Linear fc1{nullptr};
  module::GeluLinear fc2{nullptr};
};
CS_MODULE(MLP);

struct CS_API BlockImpl : module::Module {
  BlockImpl(const Scheduler &scheduler, const GPT2Config &config);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &x);
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad, const GradientSync &sync);
  module::LayerNorm ln1{nullptr}, ln2{nullptr};
  Attn attn{nullptr};
  MLP mlp{nullptr};
};
CS_MODULE(Block);

struct CS_API GPT2Impl : module::Module {
  GPT2Impl(const Scheduler &scheduler, const GPT2Config &config);
  // input_ids [B,T] int64 -> logits [B,T,padded_vocab]
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &input_ids);
  // Backward from d(logits); pairs with forward().
  void backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_logits, const GradientSync &sync = {});
  // input_ids, labels [B,T] int64 -> mean cross-entropy (fp32 scalar); fused classifier path.
  Tensor forward_loss(const Scheduler &scheduler, const ReadOnlyTensor &input_ids, const ReadOnlyTensor &labels);
  // Backward of forward_loss (the loss gradient is 1; scale through the optimizer's grad_scale).
  void backward_loss(const Scheduler &scheduler, const GradientSync &sync = {});
  [[nodiscard]] const GPT2Config &config() const { return config_; }

  module::Embedding wte{nullptr}, wpe{nullptr};
  std::vector<Block> h;
  module::LayerNorm lnf{nullptr};
  module::Linear lm_head{nullptr};

 private:
  Tensor embed(const Scheduler &scheduler, const ReadOnlyTensor &input_ids);
  void backward_trunk(const Scheduler &scheduler, Tensor grad, const GradientSync &sync);
  GPT2Config config_;
  std::shared_ptr<compute::LinearCrossEntropy::State> lce_state_;
  std::shared_ptr<compute::CrossEntropy::State> ce_state_;
  Tensor positions_;
  bool fused_embedding_{false};
  int64_t last_batch_{0}, last_seq_{0};
};
CS_MODULE(GPT2);
}  // namespace cs::models
