// SPDX-License-Identifier: Apache-2.0
// Data-parallel GPT-2 training, one process per GPU (counterpart of the reference project's
// example/gpt2/gpt2_ddp.cpp). Launch with torchrun-style environment variables (RANK,
// WORLD_SIZE, LOCAL_RANK, MASTER_ADDR, MASTER_PORT), e.g. through examples/launch.py.
// Gradients are queued into a byte-threshold bucket right after each weight gradient is
// produced on the last micro-step and all-reduced on the comm stream while backward continues;
// the bucket is flushed before the optimizer step and the average is folded into the update.
//
//   gpt2_ddp [--model 124M] [--steps N] [--micro-batch B] [--bucket-mb 25] [--backend nccl|nvp2p]
#include <cuda_runtime.h>

#include <chrono>
#include <iostream>

#include "cs/data.h"
#include "cs/models.h"
#include "cs/parallel.h"

int main(int argc, char **argv) {
  std::string model_name = "124M", backend = "nvp2p";
  int64_t steps = 10, micro_batch = 16;
  double bucket_mb = 25;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i], v = argv[i + 1];
    if (k == "--model") model_name = v;
    else if (k == "--steps") steps = std::stoll(v);
    else if (k == "--micro-batch") micro_batch = std::stoll(v);
    else if (k == "--bucket-mb") bucket_mb = std::stod(v);
    else if (k == "--backend") backend = v;
  }
  const char *lr_env = std::getenv("LOCAL_RANK");
  const int local_rank = lr_env ? std::atoi(lr_env) : 0;
  cs::DynamicScheduler scheduler{local_rank};
  CS_ASSERT_TRUE(scheduler.device().is_cuda(), "gpt2_ddp needs GPUs");
  CS_CHECK_CUDART(cudaSetDevice(local_rank));
  auto comm = cs::communication::get_comm_world(backend == "nccl" ? cs::communication::kNCCL : cs::communication::kNVP2P);
  const int64_t world = comm.get_size(), rank = comm.get_rank();

  cs::manual_seed(1234);  // identical initial weights on every rank
  cs::models::GPT2Config config = model_name == "350M"   ? cs::models::GPT2Config::gpt2_350m()
                                  : model_name == "774M" ? cs::models::GPT2Config::gpt2_774m()
                                  : model_name == "tiny" ? cs::models::GPT2Config::tiny()
                                                         : cs::models::GPT2Config::gpt2_124m();
  cs::models::GPT2 model{scheduler, config};
  std::shared_ptr<cs::module::FlatParameters> flat;
  if (backend != "nccl" && world > 1) {
    cs::communication::create_symmetric_context(comm, config.parameter_count() * 6 + (256ll << 20));
    flat = cs::parallel::flatten_symmetric(scheduler, *model, comm);
  } else {
    flat = cs::module::flatten_parameters(scheduler, *model, cs::module::FlattenOptions{}.lp_dtype(at::kBFloat16));
  }
  cs::module::AdamW optimizer{scheduler, *model, flat,
                              cs::optimizer::AdamW::Options{}.lr(3e-4).beta1(0.9).beta2(0.95).weight_decay(0.1)};
  optimizer->set_grad_scale(1.0 / static_cast<double>(world));
  cs::communication::AllReduceBucket bucket{static_cast<int64_t>(bucket_mb * (1 << 20)), cs::communication::kSUM};
  cs::models::GradientSync sync{comm, &bucket, true};
  const int64_t seq = config.block_size();
  cs::data::SyntheticDataLoader loader{micro_batch, seq, config.vocab_size(), static_cast<uint64_t>(100 + rank)};

  for (int64_t step = 0; step < steps; ++step) {
    const auto t0 = std::chrono::steady_clock::now();
    auto batch = loader.load(scheduler);
    cs::Tensor loss;
    {
      cs::autocast::ContextGuard guard{scheduler, at::kBFloat16};
      loss = model->forward_loss(scheduler, batch["input_ids"], batch["labels"]);
    }
    model->backward_loss(scheduler, sync);
    bucket.sync(scheduler, comm);
    optimizer->step(scheduler);
    optimizer->zero_grad(scheduler);
    cs::communication::AllReduce::run_inplace(scheduler, comm, {loss}, cs::communication::kAVG);
    const double value = cs::memory::to_torch(scheduler, loss).item<double>();
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (rank == 0)
      std::printf("step %4ld/%ld | loss %.6f | %.2f ms | %.0f tok/s (all ranks)\n", static_cast<long>(step + 1),
                  static_cast<long>(steps), value, dt * 1e3, static_cast<double>(micro_batch * seq * world) / dt);
  }
  scheduler.impl()->synchronize();
  cs::communication::finalize();
  return 0;
}
