// SPDX-License-Identifier: Apache-2.0
// NCCL process-group construction (kept in its own translation unit because it needs the
// NCCL headers that match the libtorch build).
#include <torch/csrc/distributed/c10d/ProcessGroupNCCL.hpp>

#include "cs/communication.h"

namespace cs::communication {
c10::intrusive_ptr<c10d::Backend> create_nccl_backend(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size) {
  auto options = c10d::ProcessGroupNCCL::Options::create();
  auto pg = c10::make_intrusive<c10d::ProcessGroupNCCL>(store, rank, size, options);
  return pg;
}
}  // namespace cs::communication
