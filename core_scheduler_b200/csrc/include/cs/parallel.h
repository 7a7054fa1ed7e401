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
}  // namespace cs::parallel
