// SPDX-License-Identifier: Apache-2.0
// A very small test harness for the C++ test programs (the image has no GoogleTest): tests register
// themselves at static-initialisation time, failures are recorded and reported per test, exceptions
// count as failures, and the process exit code is the number of failed tests.
//
//   CS_TEST(Linear, ForwardBackwardFloat32) { EXPECT_TRUE(...); EXPECT_CLOSE(a, b, rtol, atol); }
//   int main(int argc, char **argv) { return cs_test::run_all(argc, argv); }      [--filter SUBSTRING]
// Options come in "--name value" pairs; run_all reads --filter and ignores the others.
#pragma once
#include <ATen/ATen.h>

#include <atomic>
#include <cstdio>
#include <exception>
#include <functional>
#include <string>
#include <vector>

namespace cs_test {
struct Case {
  std::string name;
  std::function<void()> body;
};
inline std::vector<Case> &registry() {
  static std::vector<Case> cases;
  return cases;
}
inline std::atomic<int> &failures_of_current() {  // atomic: a test body may run on several rank threads at once
  static std::atomic<int> n{0};
  return n;
}
struct Registrar {
  Registrar(const char *suite, const char *name, std::function<void()> body) {
    registry().push_back({std::string(suite) + "." + name, std::move(body)});
  }
};
inline void report(bool ok, const char *file, int line, const std::string &what) {
  if (ok) return;
  ++failures_of_current();
  std::printf("  %s:%d: %s\n", file, line, what.c_str());
}
// max |a - b| and the bound it had to meet, for the failure message
inline std::string difference(const at::Tensor &a, const at::Tensor &b) {
  if (a.sizes() != b.sizes()) return "shapes differ";
  const auto x = a.detach().to(at::kCPU, at::kDouble), y = b.detach().to(at::kCPU, at::kDouble);
  return "max abs difference " + std::to_string((x - y).abs().max().item<double>()) + ", max |reference| " +
         std::to_string(y.abs().max().item<double>());
}
inline bool close(const at::Tensor &a, const at::Tensor &b, double rtol, double atol) {
  if (a.sizes() != b.sizes()) return false;
  return at::allclose(a.detach().to(at::kCPU, at::kDouble), b.detach().to(at::kCPU, at::kDouble), rtol, atol);
}
// Runs a test body and turns an exception into a recorded failure (also used by rank threads).
inline void guarded(const std::function<void()> &body) {
  try {
    body();
  } catch (const std::exception &e) {
    report(false, "exception", 0, e.what());
  }
}
// `runner` executes a test body; the default calls it on this thread, a multi-rank program passes one that runs it
// on every rank thread.
inline int run_all(int argc, char **argv, const std::function<void(const std::function<void()> &)> &runner = guarded) {
  std::string filter;
  for (int i = 1; i + 1 < argc; i += 2)
    if (std::string(argv[i]) == "--filter") filter = argv[i + 1];
  int ran = 0, failed = 0;
  for (auto &c : registry()) {
    if (!filter.empty() && c.name.find(filter) == std::string::npos) continue;
    std::printf("[ RUN    ] %s\n", c.name.c_str());
    std::fflush(stdout);
    failures_of_current() = 0;
    runner(c.body);
    ++ran;
    if (failures_of_current() > 0) ++failed;
    std::printf("[ %s ] %s\n", failures_of_current() > 0 ? "FAILED" : "    OK", c.name.c_str());
  }
  std::printf("%d tests ran, %d failed\n", ran, failed);
  std::fflush(stdout);
  return failed;
}
}  // namespace cs_test

#define CS_TEST(suite, name)                                                                  \
  static void cs_test_##suite##_##name();                                                     \
  static cs_test::Registrar cs_test_reg_##suite##_##name{#suite, #name, cs_test_##suite##_##name}; \
  static void cs_test_##suite##_##name()
#define EXPECT_TRUE(cond) cs_test::report(static_cast<bool>(cond), __FILE__, __LINE__, "expected: " #cond)
#define EXPECT_CLOSE(a, b, rtol, atol) \
  cs_test::report(cs_test::close((a), (b), (rtol), (atol)), __FILE__, __LINE__, std::string(#a " vs " #b ": ") + cs_test::difference((a), (b)))
