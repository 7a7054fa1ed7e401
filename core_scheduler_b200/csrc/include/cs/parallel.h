// SPDX-License-Identifier: Apache-2.0
// Parallel training strategies built on the communication layer.
//
// The reference project implements data parallelism only (bucketed all-reduce driven from the
// model's backward, example/gpt2/gpt2_ddp.cpp:341-346,630-631) and lists ZeRO and tensor
// parallelism as future work (README.md:43-47). Here:
//   * data parallel: GradientSync + AllReduceBucket (cs/models.h, cs/communication.h), with the
//     gradient arena in symmetric memory the bucket all-reduce is this library's peer-memory kernel;
//   * ZeRO: ZeroAdamW shards the fp32 master weights and the AdamW moments across ranks (block-interleaved) and
//     performs gradient reduce-scatter + AdamW + bf16 parameter all-gather as ONE kernel per bucket over peer memory,
//     overlapped with the backward pass;
//   * tensor parallel: column/row-parallel Linear with sequence-parallel activations.
#pragma once
#include "cs/communication.h"
#include "cs/models.h"
#include "cs/optimizer.h"
#include "cs/symmetric.h"

namespace cs::parallel {
// Flattens `module` with its gradient and bf16 working-copy arenas inside the communicator's
// symmetric memory, so that collectives read and write them in place. The arena length is
// padded so that it splits evenly into `world * 128`-element shards. `first`: parameter names laid out ahead of the
// others (module::FlattenOptions::first), e.g. the parameters that tensor parallelism replicates. `unequal_shards`:
// the module's parameters differ in size between ranks (tensor-parallel shards of 20 heads over 8 ranks); every arena
// is then allocated with the largest size any rank needs, so that later symmetric allocations stay aligned.
CS_API std::shared_ptr<module::FlatParameters> flatten_symmetric(const Scheduler &scheduler, const module::Module &module,
                                                                const communication::Comm &comm,
                                                                optional<at::ScalarType> lp_dtype = at::kBFloat16,
                                                                const std::vector<std::string> &first = {},
                                                                bool unequal_shards = false);

// The largest `value` any of the `size` ranks passes under the same `prefix`, agreed on through the key/value store
// (every rank publishes its value and reads all of them). Returns `value` when there is one rank or no store.
CS_API int64_t agree_on_max(c10d::Store *store, const std::string &prefix, int rank, int size, int64_t value);

struct CS_API ZeroAdamWImpl : module::OptimizerModule {
  using Options = optimizer::AdamW::Options;
  // Ownership granularity: block j of the arenas (kBlock elements) belongs to rank j % world.
  static constexpr int64_t kBlock = 16384;
  // `flat` must come from flatten_symmetric (fp32 parameters, bf16 working copies).
  ZeroAdamWImpl(const Scheduler &scheduler, const module::Module &module, const std::shared_ptr<module::FlatParameters> &flat,
                const communication::Comm &comm, const Options &options);
  // Updates the parameters whose gradient handles are given: one kernel per contiguous arena range that reduce-scatters
  // the range's gradients, runs AdamW on the blocks this rank owns and writes the new bf16 values into every rank's
  // working copy. Driven per bucket from communication::AllReduceBucket::on_reduced (with an operation-free bucket) the
  // optimizer runs beside the backward pass; step() then handles what is left.
  void step_partial(const Scheduler &scheduler, const std::vector<Tensor> &gradients, Task::Impl::Priority priority);
  // Whatever step_partial has not covered since the last step() (everything, without buckets). Gradients are averaged over the ranks.
  void step(const Scheduler &scheduler) override;
  // All-gathers the fp32 master shards into the full fp32 parameter arena of every rank (needed before saving a model
  // checkpoint; training itself only reads the bf16 copies, and the fp32 arena is not kept current in between).
  void gather_master(const Scheduler &scheduler);
  // This rank's shards: `shard<rank>.m`, `.v` and `.master` (each shard_count() values: the rank's blocks back to back).
  [[nodiscard]] OrderedDict<std::string, Tensor> named_state_tensors() const override;
  [[nodiscard]] int64_t step_count() const override { return state_->options.t; }
  void set_step_count(int64_t t) override { state_->options.t = t; }
  [[nodiscard]] int64_t shard_count() const { return shard_count_; }

 private:
  std::shared_ptr<module::FlatParameters> flat_;
  communication::Comm comm_;
  std::shared_ptr<optimizer::AdamW::State> state_;  // moments of this rank's shard only
  Tensor master_;                                   // fp32 master weights of this rank's shard only
  int64_t shard_count_{0};
  std::unordered_map<const void *, size_t> slot_of_grad_;
  std::vector<Tensor> slot_params_;
  std::vector<char> slot_done_;
  bool step_open_{false};
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
// Symmetric buffers shared by all blocks of one tensor-parallel model (created on first use): the bf16 partial
// product awaiting its reduce-scatter and two gathered-gradient buffers used in turn.
struct TPWorkspace {
  Tensor partial;
  Tensor grad_full[2];
  int next_grad{0};
  Tensor slots[2];  // [tp, rows, n] bf16: per-source slots of the GEMM -> reduce-scatter epilogue, used in turn
  int next_slot{0};
};

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
  // Symmetric-memory path: gathered LayerNorm outputs [M, d], kept from forward to backward (the weight gradients of
  // c_attn / fc1 read them again), and the model-wide workspace.
  Tensor a_full, b_full;
  std::shared_ptr<TPWorkspace> workspace;

 private:
  bool fused_forward_{false};
  bool tiled_forward_{false};
};
CS_MODULE(TPBlock);

struct CS_API TPGPT2Impl : module::Module {
  TPGPT2Impl(const Scheduler &scheduler, const models::GPT2Config &config, const communication::Comm &comm);
  // input_ids, labels: the FULL [B, T] batch on every rank (each rank embeds only its own row shard). With the
  // vocabulary-parallel classifier (padded vocabulary divisible by 8 * tp) the result is the mean loss over all
  // rows, identical on every rank; otherwise it is this rank's mean over its own rows.
  Tensor forward_loss(const Scheduler &scheduler, const ReadOnlyTensor &input_ids, const ReadOnlyTensor &labels);
  void backward_loss(const Scheduler &scheduler, const models::GradientSync &sync);
  [[nodiscard]] const models::GPT2Config &config() const { return config_; }
  // Names of the parameters that are replicated on every rank (gradients need the all-reduce).
  [[nodiscard]] std::vector<std::string> replicated_parameters() const;
  // (first head, number of heads) owned by this rank.
  [[nodiscard]] std::pair<int64_t, int64_t> head_range() const { return {h.front()->head_begin, h.front()->local_heads}; }
  // True when lm_head is split over the vocabulary (this rank holds rows [rank * V/tp, (rank + 1) * V/tp)).
  [[nodiscard]] bool vocab_parallel() const { return vocab_parallel_; }

  module::Embedding wte{nullptr}, wpe{nullptr};
  std::vector<TPBlock> h;
  module::LayerNorm lnf{nullptr};
  module::Linear lm_head{nullptr};

 private:
  models::GPT2Config config_;
  communication::Comm comm_;
  std::shared_ptr<compute::LinearCrossEntropy::State> lce_state_;
  int64_t batch_{0}, seq_{0};
  // vocabulary-parallel classifier: lm_head holds rows [rank * V/tp, (rank + 1) * V/tp)
  bool vocab_parallel_{false};
  bool ce_fused_{false};
  std::shared_ptr<TPWorkspace> workspace_;
  Tensor lnf_full_, stats_full_;                         // persistent gathered buffers (symmetric path)
  Tensor ce_logits_, ce_lse_, ce_input_;                 // kept from forward_loss to backward_loss
  ReadOnlyTensor ce_labels_;
};
CS_MODULE(TPGPT2);

// ---- the fused tensor-parallel kernels on plain tensors (one rank, current stream) ------------------------------
// What TPBlock runs inside its tasks, usable on their own (and with the single-GPU loopback contexts of
// cs/symmetric.h, where one rank at a time is emulated).
struct GatherSignal {
  uint32_t epoch{0};               // value the chunk flags reach
  const uint32_t *flags{nullptr};  // word [owner * 8 + chunk] in this rank's signal pad
  int chunks{0};
};
// all-gather of [rows, k] shards into `full` ([size * rows, k], in the arena) in `chunks` row chunks, each announced by a flag.
CS_API GatherSignal gather_rows_chunked(communication::SymmetricContext &ctx, const at::Tensor &shard, const at::Tensor &full, int chunks);
// y = full * W^T (or full * W when weight_is_rhs) by the GEMM whose loads wait for the chunk flags of `signal`;
// second tensor: GELU(y) for kEpiGeluDual. `epilogue` is a kernels::kEpi* value; `aux` the pre-activation for kEpiDGelu.
CS_API std::pair<at::Tensor, at::Tensor> gemm_on_gathered_chunks(communication::SymmetricContext &ctx, const at::Tensor &full, const at::Tensor &weight,
                                                                 bool weight_is_rhs, int epilogue, const at::Tensor &aux, const GatherSignal &signal);
// GEMM -> reduce-scatter, first half: the epilogue stores this rank's partial rows (bf16) into slot `rank` of every owner's
// `slots` ([size, rows / size, n], in the arena).
CS_API void gemm_scatter_to_slots(communication::SymmetricContext &ctx, const at::Tensor &x, const at::Tensor &weight, bool weight_is_rhs,
                                  const at::Tensor &slots);
// Second half: cross-rank barrier, then out = sum of the local slots (+ residual).
CS_API at::Tensor sum_slots(communication::SymmetricContext &ctx, const at::Tensor &slots, const at::Tensor &residual);

// Launches of this library's tensor-parallel collective kernels so far (row gathers and switch reduce-scatters on
// symmetric memory); 0 means the generic collectives were used.
CS_API int64_t fused_tp_launches();

// Row-shard collectives used by the TP model (comm-stream tasks):
// gathers [M/tp, d] row shards into [M, d];
CS_API Tensor all_gather_rows(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &shard);
// sums [M, d] partials over ranks and keeps this rank's [M/tp, d] rows (+ residual when given).
CS_API Tensor reduce_scatter_rows(const Scheduler &scheduler, const communication::Comm &comm, const ReadOnlyTensor &full,
                                  const ReadOnlyTensor *residual = nullptr);
}  // namespace cs::parallel
