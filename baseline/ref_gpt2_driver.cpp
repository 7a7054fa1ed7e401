// SPDX-License-Identifier: Apache-2.0
// Benchmark driver for the reference library (TheCoreTeam/core_scheduler) built unmodified into
// baseline/_ref/libcore_scheduler_core.so: GPT-2 training steps written against the reference's
// PUBLIC headers only (module::Linear / LayerNorm / Embedding, compute::GeLU,
// ScaledDotProductFlashAttention, CrossEntropy, Utils, module::AdamW, DynamicScheduler,
// autocast::ContextGuard, AllReduceBucket), on synthetic uniform tokens with N(0, 0.02) weights,
// fp32 parameters under a bf16 autocast guard. Nothing of core_scheduler_b200 is linked here.
// The reference's own example programs are hard-coded to one configuration and a dataset path;
// this program takes the model size, micro-batch and step counts from the command line instead.
//
//   ref_gpt2 --model 124M --micro-batch 16 --seq 1024 --steps 20 --warmup 5 [--bucket-mb 25] [--dataset DIR]
//
// One process per GPU (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_PORT in the environment; the MPI
// calls of the library are served by baseline/shims). Rank 0 prints one line
//   REF_RESULT ms_per_step=<device time, max over ranks> tokens_per_s=<all ranks> final_loss=<value>
// and, when --dataset names a directory of Parquet files with list<int64> columns input_ids and labels, a
// second line for the same steps fed by the library's own data path (LlmDataset + LlmDataLoader: a worker
// thread fills pinned host buffers, a loader task copies them to the device) with the loss read back to the
// host after every step, timed by the host clock between two full synchronisations:
//   REF_E2E ms_per_step=<max over ranks> tokens_per_s=<all ranks> h2d_bytes=<per step> d2h_bytes=<per step>
#include <arrow/compute/initialize.h>
#include <cuda_runtime.h>
#include <mpi.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "autocast.h"
#include "communication/all_reduce.h"
#include "communication/communication.h"
#include "compute/cross_entropy.h"
#include "compute/gelu.h"
#include "compute/scaled_dot_product_attention.h"
#include "compute/utils.h"
#include "data/dataloader.h"
#include "data/dataset.h"
#include "memory/to_torch.h"
#include "module/adamw.h"
#include "module/embedding.h"
#include "module/layer_norm.h"
#include "module/linear.h"
#include "module/module.h"
#include "random.h"
#include "threading/dynamic_scheduler.h"

namespace {
bool g_debug = false;
std::atomic<bool> g_e2e_done{false};
void mark(const char *what) {  // REF_DEBUG=1: progress marks on stderr (the reference aborts rather than throws)
  if (g_debug) std::fprintf(stderr, "[ref_gpt2] %s\n", what), std::fflush(stderr);
}
struct Config {
  int64_t n_layer = 12, n_head = 12, n_embd = 768, vocab = 50304, valid_vocab = 50257, seq = 1024, batch = 16;
  at::Device device{at::kCUDA, 0};
};

struct GradientQueue {  // data-parallel: gradients go into the byte-threshold bucket as they are produced
  const cs::communication::Comm *comm = nullptr;
  const cs::communication::AllReduceBucket *bucket = nullptr;
  int64_t threshold = 0;
  mutable int64_t pending = 0;  // bytes the bucket still holds (same rule as the library: flush at >= threshold)
  void push(const cs::Scheduler &s, const cs::Tensor &g, int64_t elements) const {
    if (!bucket) return;
    bucket->push_back(s, *comm, g);
    pending += elements * 4;  // fp32 gradients
    if (pending >= threshold) pending = 0;
  }
  // The library's sync() concatenates its pending list and throws on an empty one, so it is only called
  // when something is pending.
  void flush(const cs::Scheduler &s) const {
    if (bucket && pending > 0) bucket->sync(s, *comm);
    pending = 0;
  }
};

cs::compute::Linear::Options linear_options(const Config &c, int64_t in, int64_t out) {
  return cs::compute::Linear::Options{in, out}.bias(false).device(c.device).dtype(at::kFloat);
}

struct Layer : cs::module::Module {
  const Config &cfg;
  cs::module::LayerNorm ln1{nullptr}, ln2{nullptr};
  cs::module::Linear qkv{nullptr}, proj{nullptr}, fc1{nullptr}, fc2{nullptr};
  std::shared_ptr<cs::compute::ScaledDotProductFlashAttention::State> attention;
  std::shared_ptr<cs::compute::GeLU::State> gelu;

  Layer(const cs::Scheduler &s, const Config &c) : cfg{c} {
    const auto ln = cs::compute::LayerNorm::Options{{c.n_embd}}.device(c.device).dtype(at::kFloat);
    ln1 = register_module("ln1", cs::module::LayerNorm{s, ln});
    qkv = register_module("c_attn", cs::module::Linear{s, linear_options(c, c.n_embd, 3 * c.n_embd)});
    proj = register_module("c_proj", cs::module::Linear{s, linear_options(c, c.n_embd, c.n_embd)});
    ln2 = register_module("ln2", cs::module::LayerNorm{s, ln});
    fc1 = register_module("fc1", cs::module::Linear{s, linear_options(c, c.n_embd, 4 * c.n_embd)});
    fc2 = register_module("fc2", cs::module::Linear{s, linear_options(c, 4 * c.n_embd, c.n_embd)});
    attention = cs::compute::ScaledDotProductFlashAttention::init(
        s, cs::compute::ScaledDotProductFlashAttention::Options{}.is_causal(true));
    gelu = cs::compute::GeLU::init(s);
    for (auto *w : {&qkv, &proj, &fc1, &fc2}) cs::compute::Utils::normal_(s, (*w)->state()->forward.weight, 0.0, 0.02);
  }

  cs::Tensor forward(const cs::Scheduler &s, const cs::Tensor &x) {
    namespace U = cs::compute::Utils;
    const int64_t B = cfg.batch, T = cfg.seq, H = cfg.n_head, D = cfg.n_embd / cfg.n_head;
    auto parts = U::split(s, qkv->forward(s, ln1->forward(s, x)), cfg.n_embd, -1);
    auto q = U::view(s, parts[0], {B, T, H, D}), k = U::view(s, parts[1], {B, T, H, D}), v = U::view(s, parts[2], {B, T, H, D});
    auto ctx = cs::compute::ScaledDotProductFlashAttention::forward(s, attention, q, k, v);
    auto x1 = U::add(s, x, proj->forward(s, U::view(s, ctx, {B, T, cfg.n_embd})));
    auto h = cs::compute::GeLU::forward(s, gelu, fc1->forward(s, ln2->forward(s, x1)));
    return U::add(s, x1, fc2->forward(s, h));
  }

  cs::Tensor backward(const cs::Scheduler &s, const cs::Tensor &dy, const GradientQueue &queue) {
    namespace U = cs::compute::Utils;
    const int64_t B = cfg.batch, T = cfg.seq, H = cfg.n_head, D = cfg.n_embd / cfg.n_head;
    const int64_t d = cfg.n_embd;
    auto linear_backward = [&](const cs::module::Linear &layer, const cs::Tensor &grad, int64_t elements) {
      auto dx = layer->backward_input(s, grad);  // main stream
      layer->backward_parameter(s, grad);        // assist stream
      queue.push(s, layer->state()->forward.grad_weight, elements);
      return dx;
    };
    auto norm_backward = [&](const cs::module::LayerNorm &layer, const cs::Tensor &grad) {
      auto dx = layer->backward(s, grad);
      queue.push(s, layer->state()->forward.grad_weight, d);
      queue.push(s, layer->state()->forward.grad_bias, d);
      return dx;
    };
    mark(" mlp backward");
    auto dh = cs::compute::GeLU::backward(s, gelu, linear_backward(fc2, dy, 4 * d * d));
    auto dx1 = U::add(s, norm_backward(ln2, linear_backward(fc1, dh, 4 * d * d)), dy);
    mark(" attention backward");
    auto dctx = U::view(s, linear_backward(proj, dx1, d * d), {B, T, H, D});
    auto dqkv = cs::compute::ScaledDotProductFlashAttention::backward(s, attention, dctx);
    auto packed = U::cat(s,
                         {U::view(s, dqkv[0], {B, T, cfg.n_embd}), U::view(s, dqkv[1], {B, T, cfg.n_embd}),
                          U::view(s, dqkv[2], {B, T, cfg.n_embd})},
                         -1);
    return U::add(s, norm_backward(ln1, linear_backward(qkv, packed, 3 * d * d)), dx1);
  }
};

struct Model : cs::module::Module {
  const Config &cfg;
  cs::module::Embedding wte{nullptr}, wpe{nullptr};
  std::vector<std::shared_ptr<Layer>> layers;
  cs::module::LayerNorm lnf{nullptr};
  cs::module::Linear lm_head{nullptr};
  std::shared_ptr<cs::compute::CrossEntropy::State> loss_state;

  Model(const cs::Scheduler &s, const Config &c) : cfg{c} {
    wte = register_module("wte", cs::module::Embedding{s, cs::compute::Embedding::Options{c.vocab, c.n_embd}.device(c.device).dtype(at::kFloat)});
    wpe = register_module("wpe", cs::module::Embedding{s, cs::compute::Embedding::Options{c.seq, c.n_embd}.device(c.device).dtype(at::kFloat)});
    for (int64_t i = 0; i < c.n_layer; ++i) {
      layers.push_back(std::make_shared<Layer>(s, c));
      register_module(std::to_string(i), layers.back());
    }
    lnf = register_module("lnf", cs::module::LayerNorm{s, cs::compute::LayerNorm::Options{{c.n_embd}}.device(c.device).dtype(at::kFloat)});
    lm_head = register_module("lm_head", cs::module::Linear{s, linear_options(c, c.n_embd, c.vocab)});
    loss_state = cs::compute::CrossEntropy::init(s);
    cs::compute::Utils::normal_(s, wte->state()->forward.weight, 0.0, 0.02);
    cs::compute::Utils::normal_(s, wpe->state()->forward.weight, 0.0, 0.02);
    cs::compute::Utils::normal_(s, lm_head->state()->forward.weight, 0.0, 0.02);
  }

  cs::Tensor forward(const cs::Scheduler &s, const cs::Tensor &tokens, const cs::Tensor &labels) {
    namespace U = cs::compute::Utils;
    const int64_t B = cfg.batch, T = cfg.seq;
    auto positions = U::arange(s, 0, T, at::TensorOptions{}.dtype(at::kLong).device(cfg.device));
    auto x = U::add(s, wte->forward(s, tokens), U::broadcast_to(s, wpe->forward(s, positions), {B, T, cfg.n_embd}));
    for (auto &layer : layers) x = layer->forward(s, x);
    auto logits = lm_head->forward(s, lnf->forward(s, x));
    return cs::compute::CrossEntropy::forward(s, loss_state, U::view(s, logits, {B * T, cfg.vocab}), labels);
  }

  void backward(const cs::Scheduler &s, const GradientQueue &queue) {
    namespace U = cs::compute::Utils;
    const int64_t B = cfg.batch, T = cfg.seq;
    mark("loss backward");
    auto dlogits = U::view(s, cs::compute::CrossEntropy::backward(s, loss_state), {B, T, cfg.vocab});
    mark("lm_head backward");
    auto dx = lm_head->backward_input(s, dlogits);
    lm_head->backward_parameter(s, dlogits);
    queue.push(s, lm_head->state()->forward.grad_weight, cfg.vocab * cfg.n_embd);
    mark("lnf backward");
    dx = lnf->backward(s, dx);
    queue.push(s, lnf->state()->forward.grad_weight, cfg.n_embd);
    queue.push(s, lnf->state()->forward.grad_bias, cfg.n_embd);
    mark("layers backward");
    for (auto it = layers.rbegin(); it != layers.rend(); ++it) dx = (*it)->backward(s, dx, queue);
    mark("embedding backward");
    wpe->backward(s, U::sum(s, dx, 0));
    queue.push(s, wpe->state()->forward.grad_weight, cfg.seq * cfg.n_embd);
    wte->backward(s, dx);
    queue.push(s, wte->state()->forward.grad_weight, cfg.vocab * cfg.n_embd);
  }
};
}  // namespace

int main(int argc, char **argv) {
  std::string model_name = "124M";
  int64_t steps = 10, warmup = 3, micro_batch = 16, seq = 1024;
  double bucket_mb = 25.0;
  std::string dataset_dir;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i], v = argv[i + 1];
    if (k == "--model") model_name = v;
    else if (k == "--steps") steps = std::stoll(v);
    else if (k == "--warmup") warmup = std::stoll(v);
    else if (k == "--micro-batch") micro_batch = std::stoll(v);
    else if (k == "--seq") seq = std::stoll(v);
    else if (k == "--bucket-mb") bucket_mb = std::stod(v);
    else if (k == "--dataset") dataset_dir = v;
  }
  g_debug = std::getenv("REF_DEBUG") != nullptr;
  MPI_Init(&argc, &argv);
  int rank = 0, world = 1;
  MPI_Comm_rank(MPI_COMM_WORLD, &rank);
  MPI_Comm_size(MPI_COMM_WORLD, &world);
  const char *lr = std::getenv("LOCAL_RANK");
  const int local_rank = lr ? std::atoi(lr) : rank;
  if (cudaSetDevice(local_rank) != cudaSuccess) {
    std::fprintf(stderr, "ref_gpt2: no GPU %d\n", local_rank);
    return 3;
  }
  Config cfg;
  cfg.device = at::Device{at::kCUDA, static_cast<c10::DeviceIndex>(local_rank)};
  cfg.batch = micro_batch;
  cfg.seq = seq;
  if (model_name == "350M") { cfg.n_layer = 24; cfg.n_head = 16; cfg.n_embd = 1024; }
  if (model_name == "774M") { cfg.n_layer = 36; cfg.n_head = 20; cfg.n_embd = 1280; }
  if (model_name == "tiny") { cfg.n_layer = 2; cfg.n_head = 4; cfg.n_embd = 128; cfg.vocab = 512; cfg.valid_vocab = 512; }

  cs::DynamicScheduler scheduler{local_rank};
  cs::manual_seed(1234);  // identical initial weights on every rank
  // the optimizer module keeps a weak reference to the model, which therefore has to be shared-owned
  auto model_ptr = std::make_shared<Model>(scheduler, cfg);
  Model &model = *model_ptr;
  cs::module::AdamW optimizer{scheduler, model_ptr, cs::optimizer::AdamW::Options{}.lr(3e-4).beta1(0.9).beta2(0.95).weight_decay(0.1)};
  std::unique_ptr<cs::communication::Comm> comm;
  std::unique_ptr<cs::communication::AllReduceBucket> bucket;
  GradientQueue queue;
  if (world > 1) {
    comm = std::make_unique<cs::communication::Comm>(cs::communication::get_comm_world(cs::communication::kNCCL));
    bucket = std::make_unique<cs::communication::AllReduceBucket>(static_cast<int64_t>(bucket_mb * (1 << 20)), cs::communication::kSUM);
    queue.comm = comm.get();
    queue.bucket = bucket.get();
    queue.threshold = static_cast<int64_t>(bucket_mb * (1 << 20));
  }
  cs::manual_seed(100 + rank);  // different tokens on every rank

  cs::Tensor loss;
  auto train_on = [&](const cs::Tensor &tokens, const cs::Tensor &labels) {
    {
      cs::autocast::ContextGuard guard{scheduler, at::kBFloat16};
      loss = model.forward(scheduler, tokens, labels);
    }
    mark("forward done");
    model.backward(scheduler, queue);
    queue.flush(scheduler);
    mark("optimizer step");
    optimizer->step(scheduler);
    optimizer->zero_grad(scheduler);
    mark("step done");
  };
  auto one_step = [&] {
    namespace U = cs::compute::Utils;
    // uniform token ids; the labels are the same stream shifted by one position
    auto ids = U::randint(scheduler, 0, cfg.valid_vocab, {cfg.batch, cfg.seq + 1}, at::TensorOptions{}.dtype(at::kLong).device(cfg.device));
    auto tokens = U::as_strided(scheduler, ids, {cfg.batch, cfg.seq}, {cfg.seq + 1, 1}, 0);
    auto labels = U::view(scheduler, U::add(scheduler, U::as_strided(scheduler, ids, {cfg.batch, cfg.seq}, {cfg.seq + 1, 1}, 1),
                                            U::zeros(scheduler, {1}, at::TensorOptions{}.dtype(at::kLong).device(cfg.device))),
                          {cfg.batch * cfg.seq});
    train_on(tokens, labels);
  };

  for (int64_t i = 0; i < warmup; ++i) one_step();
  loss.wait();
  cudaDeviceSynchronize();
  MPI_Barrier(MPI_COMM_WORLD);
  cudaEvent_t begin, end;
  cudaEventCreate(&begin);
  cudaEventCreate(&end);
  cudaEventRecord(begin, nullptr);  // every stream is idle here: the event marks "now" on the device
  for (int64_t i = 0; i < steps; ++i) one_step();
  loss.wait();
  cudaDeviceSynchronize();          // every stream of the step has drained
  cudaEventRecord(end, nullptr);
  cudaEventSynchronize(end);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, begin, end);
  double per_step = static_cast<double>(ms) / static_cast<double>(steps);
  MPI_Shim_max_double(&per_step);
  const at::Tensor loss_tensor = cs::memory::to_torch(scheduler, loss);
  const double value = loss_tensor.item<double>();
  const int64_t loss_bytes = static_cast<int64_t>(loss_tensor.element_size());
  if (rank == 0)
    std::printf("REF_RESULT ms_per_step=%.6f tokens_per_s=%.3f final_loss=%.6f\n", per_step,
                static_cast<double>(cfg.batch * cfg.seq * world) / (per_step * 1e-3), value);
  std::fflush(stdout);

  if (!dataset_dir.empty()) {
    // The device-timed line above is already out. If the data path stalls (its worker threads meet the
    // caller on host barriers), this process leaves after a limit instead of holding the other ranks.
    const double limit_s = 60.0 + static_cast<double>(steps + 2) * per_step * 10.0 * 1e-3;
    std::thread([limit_s, rank] {
      const auto give_up = std::chrono::steady_clock::now() + std::chrono::duration<double>(limit_s);
      while (!g_e2e_done.load() && std::chrono::steady_clock::now() < give_up) std::this_thread::sleep_for(std::chrono::milliseconds(50));
      if (g_e2e_done.load()) return;
      std::fprintf(stderr, "ref_gpt2: rank %d: end-to-end phase exceeded %.0f s, leaving\n", rank, limit_s);
      std::fflush(stderr);
      std::_Exit(0);
    }).detach();
    mark("end-to-end phase");
    namespace U = cs::compute::Utils;
    // Arrow 21 and later keep the compute kernels that a dataset scan's projection calls in a library of their
    // own, which the program has to initialise; the reference was written before that split.
    const auto arrow_ready = arrow::compute::Initialize();
    if (!arrow_ready.ok()) std::fprintf(stderr, "ref_gpt2: arrow::compute::Initialize: %s\n", arrow_ready.ToString().c_str());
    cs::data::LlmDataset dataset{dataset_dir};
    auto loader = world > 1 ? std::make_unique<cs::data::LlmDataLoader>(dataset, *comm, cfg.batch, 1, false)
                            : std::make_unique<cs::data::LlmDataLoader>(dataset, cfg.batch, 1, false);
    auto e2e_step = [&] {
      auto data = loader->load(scheduler);  // pinned host buffers -> device, on the scheduler's main stream
      train_on(data.at("input_ids"), U::view(scheduler, data.at("labels"), {cfg.batch * cfg.seq}));
      return cs::memory::to_torch(scheduler, loss).item<double>();  // device -> host read of the step's loss
    };
    double last = 0.0;
    for (int i = 0; i < 2; ++i) last = e2e_step();
    cudaDeviceSynchronize();
    MPI_Barrier(MPI_COMM_WORLD);
    const auto t0 = std::chrono::steady_clock::now();
    for (int64_t i = 0; i < steps; ++i) last = e2e_step();
    cudaDeviceSynchronize();
    double e2e_per_step = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / static_cast<double>(steps);
    MPI_Shim_max_double(&e2e_per_step);
    if (rank == 0)
      std::printf("REF_E2E ms_per_step=%.6f tokens_per_s=%.3f h2d_bytes=%lld d2h_bytes=%lld final_loss=%.6f\n", e2e_per_step,
                  static_cast<double>(cfg.batch * cfg.seq * world) / (e2e_per_step * 1e-3),
                  static_cast<long long>(2 * cfg.batch * cfg.seq * 8), static_cast<long long>(loss_bytes), last);
    std::fflush(stdout);
    g_e2e_done.store(true);
  }
  MPI_Finalize();
  // The library offers no way to shut its NCCL process group down, and that group's destructor throws when it
  // runs during static destruction (the CUDA driver is gone by then): leave without running static destructors.
  std::fflush(stdout);
  std::fflush(stderr);
  std::_Exit(0);
}
