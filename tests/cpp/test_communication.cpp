// SPDX-License-Identifier: Apache-2.0
// Multi-rank tests of the collectives through the C++ API (the counterpart of the reference project's
// core_scheduler_communication_tests: test/test_all_reduce.cpp, test_all_gather.cpp, test_reduce_scatter.cpp,
// test_all_to_all.cpp). One process per GPU, started by examples/launch.py or torchrun (RANK, LOCAL_RANK,
// WORLD_SIZE, MASTER_ADDR, MASTER_PORT); every rank regenerates every other rank's data from its seed, so
// the expected values are computed locally. Unlike the reference's all-reduce test, the expectation here is
// the sum over all ranks' regenerated inputs, not the output compared with itself. Without a launcher the
// program runs as a single rank (on the CPU when there is no GPU) and checks the one-rank semantics.
//
//   python examples/launch.py --nproc 2 -- tests/cpp/bin/cs_b200_communication_tests [--filter SUBSTRING]
//   tests/cpp/bin/cs_b200_communication_tests --threads 4      (ranks as threads of one process, on the CPU)
#include <cuda_runtime.h>
#include <torch/torch.h>

#include <chrono>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <thread>

#include "cs/communication.h"
#include "cs/compute.h"
#include "cs/models.h"
#include "cs/parallel.h"
#include "cs_test.h"

namespace {
int env_int(const char *name, int fallback) {
  const char *v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
}
// One per rank: the process itself (launcher mode) or a thread of it (--threads N).
struct RankContext {
  std::unique_ptr<cs::DynamicScheduler> scheduler;
  cs::communication::Comm comm;
};
thread_local RankContext *g_rank = nullptr;
std::vector<cs::communication::Comm> g_doomed;  // --threads mode: a second group with a 300 ms rendezvous timeout
cs::DynamicScheduler &scheduler() { return *g_rank->scheduler; }
cs::communication::Comm &comm() { return g_rank->comm; }
at::Device device() { return scheduler().device(); }
int64_t rank() { return comm().get_rank(); }
int64_t world() { return comm().get_size(); }
at::Tensor host(const cs::ReadOnlyTensor &t) { return cs::memory::to_torch(scheduler(), t); }
// the tensor that the rank with this seed draws: generated on the CPU so that every rank can reproduce it
at::Tensor draw(int64_t seed, int64_t n, at::ScalarType dtype) {
  auto generator = at::detail::createCPUGenerator(static_cast<uint64_t>(seed));
  return at::rand({n}, generator, at::TensorOptions{}.dtype(dtype)).to(device());
}
cs::Tensor wrap(const at::Tensor &t) { return cs::Tensor::wrap(t.detach().clone()); }
const std::vector<at::ScalarType> kTypes{at::kFloat, at::kDouble};
const std::vector<int64_t> kSizes{128, 1 << 18};
}  // namespace

CS_TEST(AllReduce, SumAndAverageOfTwoTensors) {
  for (auto dtype : kTypes)
    for (auto n : kSizes)
      for (auto op : {cs::communication::kSUM, cs::communication::kAVG}) {
        auto a = wrap(draw(rank() + 1, n, dtype)), b = wrap(draw(100 + rank() + 1, n / 2, dtype));
        cs::communication::AllReduce::run_inplace(scheduler(), comm(), {a, b}, op);
        at::Tensor expect_a = at::zeros({n}, a.options()), expect_b = at::zeros({n / 2}, b.options());
        for (int64_t r = 0; r < world(); ++r) {
          expect_a += draw(r + 1, n, dtype);
          expect_b += draw(100 + r + 1, n / 2, dtype);
        }
        if (op == cs::communication::kAVG) {
          expect_a /= static_cast<double>(world());
          expect_b /= static_cast<double>(world());
        }
        EXPECT_CLOSE(host(a), expect_a, 1e-5, 1e-6);
        EXPECT_CLOSE(host(b), expect_b, 1e-5, 1e-6);
      }
}

CS_TEST(AllReduceBucket, FlushesAtTheByteThresholdAndOnSync) {
  const int64_t n = 1024;  // 4 KB per float tensor; threshold 10 KB -> a launch after every third tensor
  cs::communication::AllReduceBucket bucket{10 * 1024, cs::communication::kSUM};
  std::vector<cs::Tensor> tensors;
  for (int i = 0; i < 7; ++i) {
    tensors.push_back(wrap(draw(1000 * (i + 1) + rank(), n, at::kFloat)));
    bucket.push_back(scheduler(), comm(), tensors.back());
  }
  bucket.sync(scheduler(), comm());
  EXPECT_TRUE(bucket.launches() == 3);  // 3 + 3 tensors by threshold, the last one by sync
  for (int i = 0; i < 7; ++i) {
    at::Tensor expected = at::zeros({n}, tensors[i].options());
    for (int64_t r = 0; r < world(); ++r) expected += draw(1000 * (i + 1) + r, n, at::kFloat);
    EXPECT_CLOSE(host(tensors[i]), expected, 1e-5, 1e-6);
  }
}

CS_TEST(AllGather, EveryBlockIsItsOwnersDraw) {
  for (auto dtype : kTypes)
    for (auto n : kSizes) {
      std::vector<cs::Tensor> blocks;
      for (int64_t r = 0; r < world(); ++r) blocks.push_back(wrap(at::zeros({n}, at::TensorOptions{}.dtype(dtype).device(device()))));
      cs::communication::AllGather::run(scheduler(), comm(), {blocks}, {wrap(draw(rank() + 1, n, dtype))});
      for (int64_t r = 0; r < world(); ++r) EXPECT_CLOSE(host(blocks[r]), draw(r + 1, n, dtype), 0, 0);
    }
}

CS_TEST(ReduceScatter, MyBlockIsTheSumOfEveryRanksBlockForMe) {
  for (auto dtype : kTypes)
    for (auto n : kSizes) {
      std::vector<cs::ReadOnlyTensor> send;
      for (int64_t j = 0; j < world(); ++j) send.push_back(wrap(draw(rank() * world() + j + 1, n, dtype)));
      auto recv = wrap(at::zeros({n}, at::TensorOptions{}.dtype(dtype).device(device())));
      cs::communication::ReduceScatter::run(scheduler(), comm(), {recv}, {send}, cs::communication::kSUM);
      at::Tensor expected = at::zeros({n}, recv.options());
      for (int64_t r = 0; r < world(); ++r) expected += draw(r * world() + rank() + 1, n, dtype);
      EXPECT_CLOSE(host(recv), expected, 1e-5, 1e-6);
    }
}

CS_TEST(AllToAll, BlockFromRankJIsItsDrawForMe) {
  for (auto dtype : kTypes)
    for (auto n : kSizes) {
      std::vector<cs::ReadOnlyTensor> send;
      std::vector<cs::Tensor> recv;
      for (int64_t j = 0; j < world(); ++j) {
        send.push_back(wrap(draw(rank() * world() + j + 1, n, dtype)));
        recv.push_back(wrap(at::zeros({n}, at::TensorOptions{}.dtype(dtype).device(device()))));
      }
      cs::communication::AllToAll::run(scheduler(), comm(), recv, send);
      for (int64_t j = 0; j < world(); ++j) EXPECT_CLOSE(host(recv[j]), draw(j * world() + rank() + 1, n, dtype), 0, 0);
    }
}

CS_TEST(DataParallel, BucketedGradientSyncEqualsOneProcessOnTheWholeBatch) {
  // every rank trains on its own micro-batches with the bucketed all-reduce overlapping backward; a second model on
  // the same rank accumulates all ranks' micro-batches locally; after three AdamW steps the parameters agree
  if (device().is_cuda()) return;  // fp32 on the CPU is deterministic; the GPU variant lives in the Python tests
  static std::mutex init_mutex;  // model initialisation draws from the process-wide generator
  auto config = cs::models::GPT2Config::tiny();
  auto make = [&] {
    std::lock_guard<std::mutex> lock{init_mutex};
    cs::manual_seed(21);
    return cs::models::GPT2{scheduler(), config};
  };
  auto model = make(), reference = make();
  auto optimizer_of = [&](cs::models::GPT2 &m) {
    auto flat = cs::module::flatten_parameters(scheduler(), *m, cs::module::FlattenOptions{});
    cs::module::AdamW opt{scheduler(), *m, flat, cs::optimizer::AdamW::Options{}.lr(1e-2).beta1(0.9).beta2(0.95).weight_decay(0.1)};
    opt->set_grad_scale(1.0 / static_cast<double>(world()));
    return opt;
  };
  auto optimizer = optimizer_of(model), reference_optimizer = optimizer_of(reference);
  cs::communication::AllReduceBucket bucket{64 * 1024, cs::communication::kSUM};
  cs::models::GradientSync sync{comm(), &bucket, true};
  auto batch_of = [&](int step, int64_t r) {
    auto generator = at::detail::createCPUGenerator(static_cast<uint64_t>(1000 * step + r + 1));
    return at::randint(0, config.vocab_size(), {2, 33}, generator, at::TensorOptions{}.dtype(at::kLong));
  };
  auto forward = [&](cs::models::GPT2 &m, const at::Tensor &ids) {
    return m->forward_loss(scheduler(), wrap(ids.slice(1, 0, 32).contiguous()), wrap(ids.slice(1, 1, 33).contiguous()));
  };
  for (int step = 0; step < 3; ++step) {
    forward(model, batch_of(step, rank()));
    model->backward_loss(scheduler(), sync);
    bucket.sync(scheduler(), comm());
    optimizer->step(scheduler());
    optimizer->zero_grad(scheduler());
    for (int64_t r = 0; r < world(); ++r) {
      forward(reference, batch_of(step, r));
      reference->backward_loss(scheduler());
    }
    reference_optimizer->step(scheduler());
    reference_optimizer->zero_grad(scheduler());
  }
  auto mine = model->named_parameters(), expected = reference->named_parameters();
  for (auto &item : mine) EXPECT_CLOSE(host(item.value()), host(expected[item.key()]), 1e-4, 1e-5);
  EXPECT_TRUE(bucket.launches() >= 3);
}

CS_TEST(TensorParallel, ShardedModelTrainsOnRankThreads) {
  // sequence-parallel activations, column/row-parallel Linears: all-gather and reduce-scatter carry the activations,
  // the bucket carries the replicated parameters' gradients
  auto config = cs::models::GPT2Config::tiny();  // 4 heads
  if (device().is_cuda() || world() < 2 || config.n_head() % world() != 0) return;
  static std::mutex init_mutex;
  cs::parallel::TPGPT2 model{nullptr};
  {
    std::lock_guard<std::mutex> lock{init_mutex};
    cs::manual_seed(31);
    model = cs::parallel::TPGPT2{scheduler(), config, comm()};
  }
  auto flat = cs::module::flatten_parameters(scheduler(), *model, cs::module::FlattenOptions{});
  cs::module::AdamW optimizer{scheduler(), *model, flat, cs::optimizer::AdamW::Options{}.lr(3e-3).beta1(0.9).beta2(0.95).weight_decay(0.0)};
  optimizer->set_grad_scale(1.0 / static_cast<double>(world()));
  cs::communication::AllReduceBucket bucket{64 * 1024, cs::communication::kSUM};
  cs::models::GradientSync sync{comm(), &bucket, true};
  auto generator = at::detail::createCPUGenerator(41);  // every rank sees the whole batch
  auto ids = at::randint(0, config.vocab_size(), {2 * world(), 33}, generator, at::TensorOptions{}.dtype(at::kLong));
  auto x = wrap(ids.slice(1, 0, 32).contiguous()), y = wrap(ids.slice(1, 1, 33).contiguous());
  double first = 0, last = 0;
  for (int step = 0; step < 6; ++step) {
    auto loss = model->forward_loss(scheduler(), x, y);
    model->backward_loss(scheduler(), sync);
    bucket.sync(scheduler(), comm());
    optimizer->step(scheduler());
    optimizer->zero_grad(scheduler());
    last = host(loss).item<double>();
    if (step == 0) first = last;
  }
  EXPECT_TRUE(std::abs(first - std::log(static_cast<double>(config.vocab_size()))) < 0.4);
  EXPECT_TRUE(last < first - 0.3);
}

CS_TEST(FailureDetection, ARankThatNeverJoinsEndsTheCollectiveWithAnError) {
  // host-side only: the in-process group's rendezvous has a timeout; main() made a second group with a short one
  if (g_doomed.empty()) return;
  auto all_reduce = [&](const cs::communication::Comm &c, int64_t seed) {
    cs::communication::AllReduce::run_inplace(scheduler(), c, {wrap(draw(seed, 8, at::kFloat))}, cs::communication::kSUM);
  };
  all_reduce(comm(), 1);  // everybody is here
  if (rank() != world() - 1) {  // the last rank stays away from the next one
    bool raised = false;
    try {
      all_reduce(g_doomed[static_cast<size_t>(rank())], 2);
    } catch (const std::exception &e) {
      raised = std::string(e.what()).find("did not join") != std::string::npos || std::string(e.what()).find("broken") != std::string::npos;
    }
    EXPECT_TRUE(raised);
  }
  all_reduce(comm(), 3);  // the healthy group is unaffected
}

CS_TEST(FailureDetection, ASlowRankOnlyDelaysTheOthers) {
  if (comm().impl()->type != cs::communication::kTHREADS || world() < 2) return;
  if (rank() == 0) cs::communication::set_thread_comm_delay(comm(), 100);
  const auto t0 = std::chrono::steady_clock::now();
  auto x = wrap(draw(rank() + 1, 16, at::kFloat));
  cs::communication::AllReduce::run_inplace(scheduler(), comm(), {x}, cs::communication::kSUM);
  const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  at::Tensor expected = at::zeros({16});
  for (int64_t r = 0; r < world(); ++r) expected += draw(r + 1, 16, at::kFloat);
  EXPECT_CLOSE(host(x), expected, 1e-5, 1e-6);
  EXPECT_TRUE(ms >= 90.0);  // nobody got past the rendezvous before the slow rank arrived
  if (rank() == 0) cs::communication::set_thread_comm_delay(comm(), 0);
}

int main(int argc, char **argv) {
  // one intra-op thread: reductions then add in a fixed order, so two runs of the same arithmetic agree bit for bit
  // (AdamW's normalised update turns a last-bit difference of a near-zero gradient into a visible one)
  at::set_num_threads(1);
  int threads = 0;
  for (int i = 1; i + 1 < argc; i += 2)
    if (std::string(argv[i]) == "--threads") threads = std::atoi(argv[i + 1]);
  if (threads > 0) {
    // every rank is a thread of this process with a CPU scheduler of its own; collectives go through shared memory
    auto comms = cs::communication::create_thread_comms(threads);
    g_doomed = cs::communication::create_thread_comms(threads, 300);
    std::vector<RankContext> ranks(static_cast<size_t>(threads));
    for (int r = 0; r < threads; ++r) {
      ranks[static_cast<size_t>(r)].scheduler = std::make_unique<cs::DynamicScheduler>(0, cs::DynamicScheduler::Options{}.device_type(at::kCPU));
      ranks[static_cast<size_t>(r)].comm = comms[static_cast<size_t>(r)];
    }
    std::printf("%d rank threads on cpu\n", threads);
    return cs_test::run_all(argc, argv, [&](const std::function<void()> &body) {
      std::vector<std::thread> pool;
      for (int r = 0; r < threads; ++r)
        pool.emplace_back([&, r] {
          g_rank = &ranks[static_cast<size_t>(r)];
          at::set_num_threads(1);  // the setting is per calling thread
          cs_test::guarded(body);
        });
      for (auto &t : pool) t.join();
    });
  }
  if (torch::cuda::is_available()) cudaSetDevice(env_int("LOCAL_RANK", 0));
  RankContext self;
  self.scheduler = std::make_unique<cs::DynamicScheduler>(env_int("LOCAL_RANK", 0));
  self.comm = cs::communication::get_comm_world(cs::communication::kNCCL);
  g_rank = &self;
  std::printf("rank %ld of %ld on %s\n", static_cast<long>(rank()), static_cast<long>(world()), device().str().c_str());
  const int failed = cs_test::run_all(argc, argv);
  scheduler().impl()->synchronize();
  cs::communication::finalize();
  self.comm = cs::communication::Comm{};
  return failed;
}
