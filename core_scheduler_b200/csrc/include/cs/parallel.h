// Parallel training strategies built on the communication layer.
//
// The reference project implements data parallelism only (bucketed all-reduce driven from the
// model's backward, example/gpt2/gpt2_ddp.cpp:341-346,630-631) and lists ZeRO and tensor
// parallelism as future work (README.md:43-47). Here:
//   * data parallel: GradientSync + AllReduceBucket (cs/models.h, cs/communication.h), with the
//     gradient arena in symmetric memory the bucket all-reduce is this library's peer-memory kernel;
//   * ZeRO: ZeroAdamW shards the AdamW moments across ranks and performs gradient
//     reduce-scatter + AdamW + bf16 parameter all-gather as ONE kernel over peer memory;
//   * tensor parallel: column/row-parallel Linear with sequence-parallel activations.
#pragma once
#include "cs/communication.h"
#include "cs/models.h"
#include "cs/optimizer.h"
#include "cs/symmetric.h"

namespace cs::parallel {
// Flattens `module` with its gradient and bf16 working-copy arenas inside the communicator's
// symmetric memory, so that collectives read and write them in place. The arena length is
// padded so that it splits evenly into `world * 128`-element shards.
CS_API std::shared_ptr<module::FlatParameters> flatten_symmetric(const Scheduler &scheduler, const module::Module &module,
                                                                const communication::Comm &comm,
                                                                optional<at::ScalarType> lp_dtype = at::kBFloat16);

struct CS_API ZeroAdamWImpl : module::OptimizerModule {
  using Options = optimizer::AdamW::Options;
  // `flat` must come from flatten_symmetric (fp32 parameters, bf16 working copies).
  ZeroAdamWImpl(const Scheduler &scheduler, const module::Module &module, const std::shared_ptr<module::FlatParameters> &flat,
                const communication::Comm &comm, const Options &options);
  // Comm-stream task: barrier, fused reduce-scatter + AdamW + all-gather kernel, barrier; then
  // refreshes the transposed working copies. Gradients are averaged over the ranks.
  void step(const Scheduler &scheduler) override;
  // All-gathers the fp32 master shards so that every rank holds the full fp32 parameters
  // (needed before saving a checkpoint; training itself only reads the bf16 copies).
  void gather_master(const Scheduler &scheduler);
  [[nodiscard]] OrderedDict<std::string, Tensor> named_state_tensors() const override;
  [[nodiscard]] int64_t step_count() const override { return state_->options.t; }
  void set_step_count(int64_t t) override { state_->options.t = t; }
  [[nodiscard]] int64_t shard_begin() const { return shard_begin_; }
  [[nodiscard]] int64_t shard_count() const { return shard_count_; }

 private:
  std::shared_ptr<module::FlatParameters> flat_;
  communication::Comm comm_;
  std::shared_ptr<optimizer::AdamW::State> state_;  // moments of this rank's shard only
  int64_t shard_begin_{0}, shard_count_{0};
};
CS_MODULE(ZeroAdamW);

// ---------------------------------------------------------------------------------------
// Tensor parallelism with sequence-parallel activations (Megatron style)
// ---------------------------------------------------------------------------------------
// The B*T token rows are split evenly over the ranks between blocks ("sequence-parallel"
// region: LayerNorm, residual stream, embedding, classifier + loss all work on M/tp rows).
// Entering a column-parallel Linear (c_attn, fc1; output features split over ranks, attention
// heads split over ranks) the rows are all-gathered; leaving a row-parallel Linear (c_proj,
// fc2; input features split) the partial outputs are reduce-scattered back to row shards and
// the residual is added. Backward mirrors this (all-gather <-> reduce-scatter). Parameters of
// the sharded Linears are rank-local; LayerNorm, embedding and classifier parameters are
// replicated and their gradients are summed over the ranks through the all-reduce bucket.
// n_head must be divisible by the number of ranks, and so must B*T.
struct CS_API TPBlockImpl : module::Module {
  TPBlockImpl(const Scheduler &scheduler, const models::GPT2Config &config, const communication::Comm &comm);
  Tensor forward(const Scheduler &scheduler, const ReadOnlyTensor &x_shard, int64_t batch, int64_t seq);
  Tensor backward(const Scheduler &scheduler, const ReadOnlyTensor &grad_shard, const models::GradientSync &sync);
  module::LayerNorm ln1{nullptr}, ln2{nullptr};
  module::Linear c_attn{nullptr}, c_proj{nullptr}, fc1{nullptr};
  module::GeluLinear fc2{nullptr};
  std::shared_ptr<compute::ScaledDotProductAttention::State> attn_state;
  communication::Comm comm;
  // Heads [head_begin, head_begin + local_heads) live on this rank. When n_head is not a multiple of the
  // tensor-parallel size the first (n_head % tp) ranks own one head more (GPT-2 774M: 20 heads over 8 ranks = 3,3,3,3,2,2,2,2).
  int64_t local_heads{0};
  int64_t head_begin{0};
  Tensor saved_ln1_out, saved_ln2_out;  // row shards kept for the backward re-gather (fused path)
};
CS_MODULE(TPBlock);

struct CS_API TPGPT2Impl : module::Module {
  TPGPT2Impl(const Scheduler &scheduler, const models::GPT2Config &config, const communication::Comm &comm);
  // input_ids, labels: the FULL [B, T] batch on every rank (each rank embeds and scores only its
  // own row shard). Returns this rank's mean loss over its rows; average over ranks for the
  // global loss.
  Tensor forward_loss(const Scheduler &scheduler, const ReadOnlyTensor &input_ids, const ReadOnlyTensor &labels);
  void backward_loss(const Scheduler &scheduler, const models::GradientSync &sync);
  [[nodiscard]] const models::GPT2Config &config() const { return config_; }
  // Names of the parameters that are replicated on every rank (gradients need the all-reduce).
  [[nodiscard]] std::vector<std::string> replicated_parameters() const;
  // (first head, number of heads) owned by this rank.
  [[nodiscard]] std::pair<int64_t, int64_t> head_range() const { return {h.front()->head_begin, h.front()->local_heads}; }

  module::Embedding wte{nullptr}, wpe{nullptr};
  std::vector<TPBlock> h;
  module::LayerNorm lnf{nullptr};
  module::Linear lm_head{nullptr};

 private:
  models::GPT2Config config_;
  communication::Comm comm_;
  std::shared_ptr<compute::LinearCrossEntropy::State> lce_state_;
  int64_t batch_{0}, seq_{0};
};
CS_MODULE(TPGPT2);

// Fused tensor-parallel paths (one tcgen05 GEMM kernel each, over peer memory):
//   all-gather -> GEMM: y[M, out_local] = gather(x_shard)[M, in] * W^T. The kernel's TMA producer
//     reads every row block of x directly from its owner's symmetric buffer, own block first.
//   GEMM -> reduce-scatter: the partial product's tiles are reduce-added (fp32) by the epilogue
//     into the accumulator of the rank that owns the rows; the owner then adds the residual and
//     rounds to bf16.
// They apply when the communicator has symmetric memory, tensors are bf16 on the GPU and
// M / tp is a multiple of 256; otherwise the unfused composition is used.
CS_API Tensor column_parallel_forward(const Scheduler &scheduler, const communication::Comm &comm,
                                      const std::shared_ptr<compute::Linear::State> &state, const ReadOnlyTensor &x_shard);
CS_API Tensor row_parallel_forward(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &weight,
                                   const ReadOnlyTensor &x, const ReadOnlyTensor *residual_shard, bool weight_is_rhs);
CS_API int64_t fused_tp_launches();

// Row-shard collectives used by the TP model (comm-stream tasks):
// gathers [M/tp, d] row shards into [M, d];
CS_API Tensor all_gather_rows(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &shard);
// sums [M, d] partials over ranks and keeps this rank's [M/tp, d] rows (+ residual when given).
CS_API Tensor reduce_scatter_rows(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &full,
                                  const ReadOnlyTensor *residual = nullptr);
}  // namespace cs::parallel
