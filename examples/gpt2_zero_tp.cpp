// SPDX-License-Identifier: Apache-2.0
// GPT-2 training with the sharded optimizer (--mode zero) or tensor + sequence parallelism
// (--mode tp), one process per GPU. The reference project has neither mode; its data-parallel
// example is example/gpt2/gpt2_ddp.cpp. Launch with torchrun-style environment variables (RANK,
// WORLD_SIZE, LOCAL_RANK, MASTER_ADDR, MASTER_PORT).
//
//   zero: gradients are written into a peer-mapped arena; one kernel per step pulls this rank's
//         gradient shard from every peer, applies AdamW to its shard of the fp32 master weights
//         and pushes the updated bf16 shard into every peer's working copy.
//   tp:   every rank sees the whole batch; QKV/fc1 are column-parallel (all-gather -> GEMM in one
//         kernel), proj/fc2 row-parallel (GEMM -> reduce-scatter in one kernel), LayerNorm and
//         residuals work on a sequence shard. Only replicated parameters use the all-reduce bucket.
//
//   gpt2_zero_tp --mode zero|tp [--model 124M|350M|774M|tiny] [--steps N] [--batch B]
//                [--metrics out.jsonl] [--save-dir DIR] [--watchdog-ms 600000]
#include <cuda_runtime.h>

#include <chrono>
#include <filesystem>
#include <iostream>

#include "cs/data.h"
#include "cs/models.h"
#include "cs/observability.h"
#include "cs/parallel.h"

int main(int argc, char **argv) {
  std::string model_name = "124M", mode = "zero", metrics_path, save_dir;
  int64_t steps = 10, batch = 16, watchdog_ms = 600000;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i], v = argv[i + 1];
    if (k == "--model") model_name = v;
    else if (k == "--mode") mode = v;
    else if (k == "--steps") steps = std::stoll(v);
    else if (k == "--batch") batch = std::stoll(v);
    else if (k == "--metrics") metrics_path = v;
    else if (k == "--save-dir") save_dir = v;
    else if (k == "--watchdog-ms") watchdog_ms = std::stoll(v);
  }
  CS_ASSERT_TRUE(mode == "zero" || mode == "tp", "--mode must be zero or tp");
  const char *lr_env = std::getenv("LOCAL_RANK");
  const int local_rank = lr_env ? std::atoi(lr_env) : 0;
  cs::DynamicScheduler scheduler{local_rank};
  CS_ASSERT_TRUE(scheduler.device().is_cuda(), "gpt2_zero_tp needs GPUs");
  CS_CHECK_CUDART(cudaSetDevice(local_rank));
  auto comm = cs::communication::get_comm_world(cs::communication::kNVP2P);
  const int64_t world = comm.get_size(), rank = comm.get_rank();
  CS_ASSERT_TRUE(world > 1, "launch at least two ranks");

  cs::manual_seed(1234);  // identical initial weights on every rank
  cs::models::GPT2Config config = model_name == "350M"   ? cs::models::GPT2Config::gpt2_350m()
                                  : model_name == "774M" ? cs::models::GPT2Config::gpt2_774m()
                                  : model_name == "tiny" ? cs::models::GPT2Config::tiny()
                                                         : cs::models::GPT2Config::gpt2_124m();
  const bool tp = mode == "tp";
  // tensor parallel: two gathered [tokens, d] bf16 activations per block stay in symmetric buffers from forward to
  // backward, plus partial-product, gradient and classifier buffers; ZeRO: fp32 gradients + bf16 copies + staging
  const int64_t tp_rows_bytes = batch * config.block_size() * config.n_embd() * 2;
  cs::communication::create_symmetric_context(
      comm, tp ? (2 * config.n_layer() + 8) * tp_rows_bytes + (320ll << 20) +
                     (config.parameter_count() / world + 2 * config.padded_vocab_size() * config.n_embd()) * 6
               : config.parameter_count() * 6 + (256ll << 20));

  cs::models::GPT2 dp_model{nullptr};
  cs::parallel::TPGPT2 tp_model{nullptr};
  std::shared_ptr<cs::module::FlatParameters> flat;
  std::shared_ptr<cs::module::OptimizerModule> optimizer;
  cs::communication::AllReduceBucket bucket{25 << 20, cs::communication::kSUM};
  cs::models::GradientSync sync;
  const auto adamw = cs::optimizer::AdamW::Options{}.lr(3e-4).beta1(0.9).beta2(0.95).weight_decay(0.1);
  if (tp) {
    tp_model = cs::parallel::TPGPT2{scheduler, config, comm};
    // gradient and working-copy arenas in symmetric memory, the replicated parameters first: their gradients are one
    // range that is all-reduced in place, and the sharded parameters are one range for the optimizer
    flat = cs::parallel::flatten_symmetric(scheduler, *tp_model, comm, at::kBFloat16, tp_model->replicated_parameters(),
                                           /*unequal_shards=*/true);
    auto opt = std::make_shared<cs::module::AdamWImpl>(scheduler, *tp_model, flat, adamw);
    opt->set_grad_scale(1.0 / static_cast<double>(world));
    optimizer = opt;
    sync = cs::models::GradientSync{comm, &bucket, true};
  } else {
    dp_model = cs::models::GPT2{scheduler, config};
    flat = cs::parallel::flatten_symmetric(scheduler, *dp_model, comm);
    auto zero = std::make_shared<cs::parallel::ZeroAdamWImpl>(scheduler, *dp_model, flat, comm, adamw);
    optimizer = zero;
    // the bucket only groups the gradients; each bucket is reduce-scattered, updated and all-gathered by one kernel while
    // the backward pass of the earlier layers is still running
    bucket.skip_reduction(true);
    bucket.on_reduced([weak = std::weak_ptr<cs::parallel::ZeroAdamWImpl>(zero)](const cs::Scheduler &s, const std::vector<cs::Tensor> &grads,
                                                                              cs::Task::Impl::Priority priority) {
      if (auto z = weak.lock()) z->step_partial(s, grads, priority);
    });
    sync = cs::models::GradientSync{comm, &bucket, true};
  }
  const int64_t seq = config.block_size();
  // tensor-parallel ranks consume the same batch; data-parallel (zero) ranks different ones
  cs::data::SyntheticDataLoader loader{batch, seq, config.vocab_size(), static_cast<uint64_t>(100 + (tp ? 0 : rank))};
  cs::metrics::MetricsLogger logger{cs::metrics::MetricsLogger::Options{}.jsonl_path(metrics_path).rank(rank)};
  cs::fault::Watchdog watchdog{comm, cs::fault::Watchdog::Options{}.timeout_ms(watchdog_ms)};
  const double tokens_per_step = static_cast<double>(batch * seq * (tp ? 1 : world));

  for (int64_t step = 0; step < steps; ++step) {
    watchdog.check();  // a stalled or failed peer is reported before the next launch
    const auto t0 = std::chrono::steady_clock::now();
    auto data = loader.load(scheduler);
    cs::Tensor loss;
    {
      cs::autocast::ContextGuard guard{scheduler, at::kBFloat16};
      loss = tp ? tp_model->forward_loss(scheduler, data["input_ids"], data["labels"])
                : dp_model->forward_loss(scheduler, data["input_ids"], data["labels"]);
    }
    if (tp) {
      tp_model->backward_loss(scheduler, sync);
      bucket.sync(scheduler, comm);
    } else {
      dp_model->backward_loss(scheduler, sync);
      bucket.sync(scheduler, comm);
    }
    optimizer->step(scheduler);
    optimizer->zero_grad(scheduler);
    cs::communication::AllReduce::run_inplace(scheduler, comm, {loss}, cs::communication::kAVG);
    cs::metrics::StepRecord record;
    record.step = step + 1;
    record.loss = cs::memory::to_torch(scheduler, loss).item<double>();
    record.lr = 3e-4;
    record.dt_host_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    record.tokens_per_sec = tokens_per_step / (record.dt_host_ms * 1e-3);
    record.mfu = cs::metrics::mfu(config.train_flops_per_token(seq), tokens_per_step, record.dt_host_ms * 1e-3,
                                  1.3287e15 * static_cast<double>(world));
    logger.log(record);
    watchdog.progress(step + 1);
  }
  if (!save_dir.empty()) {
    if (!tp) std::static_pointer_cast<cs::parallel::ZeroAdamWImpl>(optimizer)->gather_master(scheduler);
    cs::checkpoint::Meta meta;
    meta.step = steps;
    meta.lr = 3e-4;
    meta.seed = 1234;
    meta.data_cursor = steps;
    meta.world_size = world;
    meta.tp_size = tp ? world : 1;
    meta.zero = !tp;
    meta.model = model_name;
    // zero: every rank holds the full fp32 weights after gather_master, rank 0 writes the canonical
    // file; tp: every rank writes its own shard directory
    const std::string dir = tp ? save_dir + "/tp_rank" + std::to_string(rank) : save_dir;
    const cs::module::Module &m = tp ? static_cast<const cs::module::Module &>(*tp_model) : static_cast<const cs::module::Module &>(*dp_model);
    cs::checkpoint::save_training_state(scheduler, dir, m, tp ? optimizer.get() : nullptr, meta, rank, tp ? rank : 0);
    if (!tp) {
      // the sharded optimizer state: every rank writes its own blocks (master weights and both moments);
      // `python -m core_scheduler_b200.utils.checkpoint merge-zero` turns the files into per-parameter tables
      const std::string shard_dir = save_dir + "/zero_rank" + std::to_string(rank);
      std::filesystem::create_directories(shard_dir);
      cs::save(*optimizer, shard_dir + "/optimizer.parquet");
    }
  }
  watchdog.stop();
  scheduler.impl()->synchronize();
  cs::communication::finalize();
  return 0;
}
