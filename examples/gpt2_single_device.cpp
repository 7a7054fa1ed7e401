// SPDX-License-Identifier: Apache-2.0
// GPT-2 training on one device through the C++ API (counterpart of the reference project's
// example/gpt2/gpt2_single_device.cpp): fp32 master parameters, bf16 autocast on GPUs, cosine
// learning rate with warm-up, gradient accumulation, loss log as CSV. Data: a Parquet token
// dataset directory (--data DIR) or synthetic uniform token ids.
//
//   gpt2_single_device [--model tiny|124M|350M|774M] [--steps N] [--micro-batch B] [--seq T]
//                      [--grad-accum K] [--data DIR] [--log FILE] [--save FILE.parquet]
#include <chrono>
#include <cmath>
#include <cstring>
#include <fstream>
#include <iostream>

#include "cs/data.h"
#include "cs/models.h"

namespace {
struct Args {
  std::string model = "tiny", data, log, save;
  int64_t steps = 10, micro_batch = 4, seq = 64, grad_accum = 1;
  double lr = 6e-4, min_lr = 6e-5;
  int64_t warmup = 2;
};
Args parse(int argc, char **argv) {
  Args a;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i], v = argv[i + 1];
    if (k == "--model") a.model = v;
    else if (k == "--steps") a.steps = std::stoll(v);
    else if (k == "--micro-batch") a.micro_batch = std::stoll(v);
    else if (k == "--seq") a.seq = std::stoll(v);
    else if (k == "--grad-accum") a.grad_accum = std::stoll(v);
    else if (k == "--data") a.data = v;
    else if (k == "--log") a.log = v;
    else if (k == "--save") a.save = v;
    else if (k == "--lr") a.lr = std::stod(v);
  }
  return a;
}
double cosine_lr(const Args &a, int64_t step) {
  if (step < a.warmup) return a.lr * static_cast<double>(step + 1) / static_cast<double>(a.warmup);
  const double ratio = static_cast<double>(step - a.warmup) / std::max<double>(1.0, static_cast<double>(a.steps - a.warmup));
  return a.min_lr + 0.5 * (1.0 + std::cos(M_PI * ratio)) * (a.lr - a.min_lr);
}
}  // namespace

int main(int argc, char **argv) {
  const Args args = parse(argc, argv);
  cs::DynamicScheduler scheduler{0};
  const bool cuda = scheduler.device().is_cuda();
  cs::manual_seed(1337);
  cs::models::GPT2Config config = args.model == "124M"   ? cs::models::GPT2Config::gpt2_124m()
                                  : args.model == "350M" ? cs::models::GPT2Config::gpt2_350m()
                                  : args.model == "774M" ? cs::models::GPT2Config::gpt2_774m()
                                                         : cs::models::GPT2Config::tiny();
  config.scale_residual_init(true);
  cs::models::GPT2 model{scheduler, config};
  cs::module::FlattenOptions fo;
  if (cuda) fo.lp_dtype(at::kBFloat16);
  auto flat = cs::module::flatten_parameters(scheduler, *model, fo);
  cs::module::AdamW optimizer{scheduler, *model, flat,
                              cs::optimizer::AdamW::Options{}.lr(args.lr).beta1(0.9).beta2(0.95).weight_decay(0.1)};
  optimizer->set_grad_scale(1.0 / static_cast<double>(args.grad_accum));

  std::unique_ptr<cs::data::LlmDataLoader> file_loader;
  std::unique_ptr<cs::data::SyntheticDataLoader> synthetic;
  if (!args.data.empty()) {
    cs::data::LlmDataset dataset{args.data};
    file_loader = std::make_unique<cs::data::LlmDataLoader>(dataset, args.micro_batch, 1, false);
  } else {
    synthetic = std::make_unique<cs::data::SyntheticDataLoader>(args.micro_batch, std::min(args.seq, config.block_size()),
                                                                config.vocab_size(), 0);
  }
  std::ofstream log;
  if (!args.log.empty()) {
    log.open(args.log);
    log << "Step,Loss\n";
  }
  const int64_t tokens_per_step = args.micro_batch * std::min(args.seq, config.block_size()) * args.grad_accum;
  for (int64_t step = 0; step < args.steps; ++step) {
    const auto t0 = std::chrono::steady_clock::now();
    cs::Tensor loss;
    for (int64_t micro = 0; micro < args.grad_accum; ++micro) {
      auto batch = file_loader ? file_loader->load(scheduler) : synthetic->load(scheduler);
      if (cuda) {
        cs::autocast::ContextGuard guard{scheduler, at::kBFloat16};
        loss = model->forward_loss(scheduler, batch["input_ids"], batch["labels"]);
      } else {
        loss = model->forward_loss(scheduler, batch["input_ids"], batch["labels"]);
      }
      model->backward_loss(scheduler);
    }
    optimizer->set_lr(cosine_lr(args, step));
    optimizer->step(scheduler);
    optimizer->zero_grad(scheduler);
    const double value = cs::memory::to_torch(scheduler, loss).item<double>();  // one host sync per step
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::printf("step %4ld/%ld | loss %.6f | lr %.2e | %.2f ms | %.0f tok/s\n", static_cast<long>(step + 1),
                static_cast<long>(args.steps), value, optimizer->get_lr(), dt * 1e3, static_cast<double>(tokens_per_step) / dt);
    if (log.is_open()) log << step << "," << value << "\n";
  }
  if (!args.save.empty()) cs::save(*model, args.save);
  return 0;
}
